"""KV cache with the reference's interface (cache_hub/flash_attn_cache.py, cache_hub/cache.py) and a block-hybrid
variant whose host-resident part is streamed to the GPU on a side stream while decode runs.

``flash_attn_cache`` keeps the reference's methods and shapes: per layer K and V ``[B, max_len, Hkv, D]``,
on the GPU when the memory model says they fit (cache.py:45-83, flash_attn_cache.py:128-141), otherwise in
PINNED host memory (the reference's are pageable and its copies block, flash_attn_cache.py:7-19); prefill
copies run on a copy stream and are fenced with events instead of device-wide synchronisation.

``HybridKVCache`` splits every layer's sequence into blocks: the first ``gpu_fraction`` of the blocks live on
the GPU, the rest in pinned host memory.  A decode step attends to the resident part directly and to the host
part through two staging buffers that the side stream refills for the next layer while the current layer's
kernels run; the two partial results are combined by the LSE merge kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib as L
from .. import ops


def kv_memory_model(layer_num, batch_size, max_length, kv_head, num_heads, head_dim, num_gpus, model_size,
                    total_gpu_memory_gb):
    """The reference's memory budget (cache.py:45-83) and allocation decision (flash_attn_cache.py:128-141):
    returns (free_memory_gb, kv_consumption_gb, fits_on_gpu)."""
    gb = 1024.0 ** 3
    weights = model_size * 2
    per = num_heads * max_length * head_dim * 2 / gb
    prefill = per + per + (num_heads + 2 * kv_head) * max_length * head_dim * 2 / gb + 4 * per
    free = total_gpu_memory_gb - weights - prefill * num_gpus
    kv = 2 * layer_num * batch_size * max_length * kv_head * head_dim * 2 / gb
    return free, kv, free > kv * 1.3


def _copy_rows(dst: torch.Tensor, src: torch.Tensor, stream: torch.cuda.Stream):
    """dst[...] = src[...] for two [rows, row_elems]-shaped views (one pinned host, one device) through
    sqattn_cache_copy_rows on ``stream``."""
    assert dst.dim() == 2 and src.dim() == 2 and dst.shape == src.shape and dst.stride(1) == 1 and src.stride(1) == 1
    es = dst.element_size()
    L.check(L.lib.sqattn_cache_copy_rows(dst.data_ptr(), dst.stride(0) * es, src.data_ptr(), src.stride(0) * es,
                                         dst.shape[1] * es, dst.shape[0], int(dst.is_cuda), stream.cuda_stream))


class flash_attn_cache:
    """Reference-compatible cache (one device)."""

    def __init__(self, valid_start, layer_num, batch_size, max_length, num_key_value_heads, num_heads, head_dim,
                 dtype, layer_mapping=None, num_gpus=1, model_size=0, device="cuda", force_host: Optional[bool] = None):
        self.valid_start = valid_start
        self.valid_length = None          # device int64 [B]
        self.valid_length_host = None     # the same numbers on the host (no synchronisation to read them)
        self.layer_num, self.batch_size, self.max_length = layer_num, batch_size, max_length
        self.kv_head, self.num_heads, self.head_dim, self.dtype = num_key_value_heads, num_heads, head_dim, dtype
        self.context = 0
        self.device = torch.device(device)
        total_gb = torch.cuda.get_device_properties(self.device).total_memory / 1024 ** 3 * num_gpus
        self.free_memory, self.kv_consumption, fits = kv_memory_model(
            layer_num, batch_size, max_length, num_key_value_heads, num_heads, head_dim, num_gpus, model_size, total_gb)
        self.allocated = fits if force_host is None else (not force_host)
        shape = (batch_size, max_length, num_key_value_heads, head_dim)
        if self.allocated:
            self.key_cache = [torch.empty(shape, dtype=dtype, device=self.device) for _ in range(layer_num)]
            self.value_cache = [torch.empty(shape, dtype=dtype, device=self.device) for _ in range(layer_num)]
        else:
            self.key_cache = [torch.empty(shape, dtype=dtype, pin_memory=True) for _ in range(layer_num)]
            self.value_cache = [torch.empty(shape, dtype=dtype, pin_memory=True) for _ in range(layer_num)]
        self.copystream = torch.cuda.Stream(self.device)
        self.copyevents = [torch.cuda.Event() for _ in range(layer_num)]
        self.batch_indices = torch.arange(batch_size, device=self.device)

    def prefill_update_kv_cache(self, query_states, key_states, value_states, layer_idx, start_bdx):
        """Store the valid part of one sequence's K/V (flash_attn_cache.py:153-231); the copy runs on the copy
        stream after the producing stream's work and is fenced by ``sync``."""
        bsz, seq_len, _, _ = key_states.shape
        assert bsz == 1, "Multi-batch prefilling only support prefill single batch one by one."
        assert seq_len <= self.max_length, f"Prefilling sequence length {seq_len} exceeds max length {self.max_length}."
        vs = self.valid_start[start_bdx] if isinstance(self.valid_start, (tuple, list)) else self.valid_start
        vs = int(vs)
        valid = seq_len - vs
        if self.valid_length is None:
            self.valid_length = torch.full((self.batch_size,), valid, dtype=torch.int64, device=self.device)
            self.valid_length_host = [valid] * self.batch_size
        if layer_idx == 0 and self.valid_length_host[start_bdx] != valid:
            self.valid_length[start_bdx] = valid
            self.valid_length_host[start_bdx] = valid
        # a dtype conversion runs on the producing stream: it has to be enqueued BEFORE the event the copy stream waits on
        srcs = []
        for states in (key_states, value_states):
            src = states[0, vs:vs + valid]                               # may be a strided view of a fused projection
            srcs.append(src if src.dtype == self.dtype else src.to(self.dtype))
        ready = torch.cuda.Event()
        ready.record()
        self.copystream.wait_event(ready)
        for cache, src in ((self.key_cache, srcs[0]), (self.value_cache, srcs[1])):
            dst = cache[layer_idx][start_bdx, :valid]                    # [valid, Hkv, D], contiguous
            src.record_stream(self.copystream)
            if self.allocated:
                with torch.cuda.stream(self.copystream):
                    dst.copy_(src, non_blocking=True)
            else:
                _copy_rows(dst.flatten(1), src.flatten(1), self.copystream)
        self.copyevents[layer_idx].record(self.copystream)
        if layer_idx == self.layer_num - 1 and start_bdx + bsz == self.batch_size:
            self.context += seq_len
        return key_states[:, vs:], value_states[:, vs:]

    def sync(self, layer_idx, start_bdx=0):
        """Make the current stream wait for the layer's cache copies."""
        torch.cuda.current_stream().wait_event(self.copyevents[layer_idx])

    def move_gpu(self):
        """Bring a host-resident cache onto the GPU before decode (flash_attn_cache.py:143-151)."""
        if not self.allocated:
            for ldx in range(self.layer_num):
                self.copyevents[ldx].synchronize()
                self.key_cache[ldx] = self.key_cache[ldx].to(self.device, non_blocking=True)
                self.value_cache[ldx] = self.value_cache[ldx].to(self.device, non_blocking=True)
            self.allocated = True

    def decode_update_kv_cache(self, key_states, value_states, layer_idx):
        """Append one token per sequence at ``valid_length`` and return the whole layer cache
        (flash_attn_cache.py:239-256)."""
        kc, vc = self.key_cache[layer_idx], self.value_cache[layer_idx]
        kn, vn = key_states[:, 0], value_states[:, 0]                    # [B, Hkv, D], possibly views of a fused projection
        if kn.dtype != self.dtype or not kn[0].is_contiguous() or kn.data_ptr() % 16:
            kn = kn.to(self.dtype).contiguous()
        if vn.dtype != self.dtype or not vn[0].is_contiguous() or vn.data_ptr() % 16:
            vn = vn.to(self.dtype).contiguous()
        row = kc.shape[2] * kc.shape[3]
        L.check(L.lib.sqattn_cache_append(kc.data_ptr(), vc.data_ptr(), kn.data_ptr(), vn.data_ptr(),
                                          self.valid_length.data_ptr(), kc.stride(0), kc.stride(1),
                                          kn.stride(0) if kn.shape[0] > 1 else row, self.batch_size, row, kc.shape[1],
                                          torch.cuda.current_stream().cuda_stream))
        if layer_idx == self.layer_num - 1:
            self.context += 1
            self.valid_length += 1
            self.valid_length_host = [x + 1 for x in self.valid_length_host]
        return self.key_cache[layer_idx], self.value_cache[layer_idx]

    def decode_attention(self, query, layer_idx, kv_len: int, out_dtype=None):
        """Split-KV decode over the layer's cache: query [B,1,Hq,D] -> [B,1,Hq,D]."""
        return ops.decode(query, self.key_cache[layer_idx], self.value_cache[layer_idx], layout="NHD",
                          out_dtype=out_dtype or self.dtype, kv_len=kv_len)


def split_blocks(num_tokens: int, block_tokens: int, gpu_fraction: float):
    """(resident_tokens, host_tokens): whole blocks, the first round(gpu_fraction * blocks) of them resident."""
    nblocks = (num_tokens + block_tokens - 1) // block_tokens
    resident_blocks = min(nblocks, max(0, int(round(gpu_fraction * nblocks))))
    resident = min(num_tokens, resident_blocks * block_tokens)
    return resident, num_tokens - resident


class HybridKVCache:
    """Block-hybrid cache for long-context decode: [B, Hkv, tokens, D] per layer, the first part on the GPU, the
    rest in pinned host memory, staged through two device buffers by a side stream."""

    def __init__(self, layer_num, batch_size, num_tokens, num_key_value_heads, head_dim, dtype, gpu_fraction=0.25,
                 block_tokens=4096, device="cuda"):
        self.layer_num, self.batch, self.tokens = layer_num, batch_size, num_tokens
        self.hkv, self.d, self.dtype = num_key_value_heads, head_dim, dtype
        self.device = torch.device(device)
        self.resident, self.host_tokens = split_blocks(num_tokens, block_tokens, gpu_fraction)
        rs, hs = (batch_size, num_key_value_heads, self.resident, head_dim), (batch_size, num_key_value_heads, self.host_tokens, head_dim)
        self.k_res = [torch.empty(rs, dtype=dtype, device=self.device) for _ in range(layer_num)]
        self.v_res = [torch.empty(rs, dtype=dtype, device=self.device) for _ in range(layer_num)]
        self.k_host = [torch.empty(hs, dtype=dtype, pin_memory=True) for _ in range(layer_num)]
        self.v_host = [torch.empty(hs, dtype=dtype, pin_memory=True) for _ in range(layer_num)]
        self.stage = [(torch.empty(hs, dtype=dtype, device=self.device), torch.empty(hs, dtype=dtype, device=self.device))
                      for _ in range(2)]
        self.side = torch.cuda.Stream(self.device)
        self.filled = [torch.cuda.Event() for _ in range(2)]
        self.released = [torch.cuda.Event() for _ in range(2)]
        for e in self.released:
            e.record()

    def load(self, layer_idx, key, value):
        """key/value [B, Hkv, tokens, D] (any device) -> this layer's resident and host parts."""
        self.k_res[layer_idx].copy_(key[:, :, :self.resident])
        self.v_res[layer_idx].copy_(value[:, :, :self.resident])
        self.k_host[layer_idx].copy_(key[:, :, self.resident:])
        self.v_host[layer_idx].copy_(value[:, :, self.resident:])

    def prefetch(self, layer_idx):
        """Start copying the layer's host part into staging buffer layer_idx % 2 on the side stream."""
        if self.host_tokens == 0:
            return
        slot = layer_idx % 2
        self.side.wait_event(self.released[slot])  # the previous user of the slot has finished reading it
        rows = self.batch * self.hkv * self.host_tokens
        for dst, src in ((self.stage[slot][0], self.k_host[layer_idx]), (self.stage[slot][1], self.v_host[layer_idx])):
            _copy_rows(dst.view(rows, self.d), src.view(rows, self.d), self.side)
        self.filled[slot].record(self.side)

    def decode_attention(self, query, layer_idx, prefetch_next=True, out_dtype=None):
        """query [B,Hq,1,D] -> O [B,Hq,1,D]; the next layer's host part is fetched while this layer computes."""
        b, hq, _, d = query.shape
        cur = torch.cuda.current_stream()
        if prefetch_next and layer_idx + 1 < self.layer_num:
            self.prefetch(layer_idx + 1)
        parts = []
        if self.resident:
            parts.append(ops.decode(query, self.k_res[layer_idx], self.v_res[layer_idx], partial=True))
        if self.host_tokens:
            slot = layer_idx % 2
            cur.wait_event(self.filled[slot])
            parts.append(ops.decode(query, self.stage[slot][0], self.stage[slot][1], partial=True))
            self.released[slot].record(cur)
        po = torch.stack([p[0].reshape(b * hq, d) for p in parts])
        pl = torch.stack([p[1].reshape(b * hq) for p in parts])
        return ops.decode_merge(po, pl, out_dtype=out_dtype or self.dtype).view(b, hq, 1, d)
