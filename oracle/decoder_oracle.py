"""TEST INFRASTRUCTURE ONLY — CPU restatement of the reference's decoder-layer glue around the attention operator.

Nothing shipped imports this file.  It restates, in torch-CPU tensor ops of the activation dtype (every op
rounds its result to that dtype, as Paddle's eager ops do), the pieces of the reference runtime that call the
attention operator:

* ``rmsnorm``, ``silu_and_mul``, ``apply_rope`` — model_hub/utils.py:4-18, 20-106
* ``layer_prefill`` / ``layer_decode`` — model_hub/LLM.py:40-116 (with model_hub/qwen.py:292-379 for the
  projections)

Parity unpinned: the reference's runtime needs Paddle and a checkpoint, neither of which is available, and it
has no golden vectors; the op-by-op rounding of Paddle's bf16 kernels is assumed to be round-to-nearest of an
fp32 result.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def silu_and_mul(hidden_states: torch.Tensor) -> torch.Tensor:
    """model_hub/utils.py:4-12"""
    x1, x2 = hidden_states.chunk(2, dim=-1)
    return x2 * (x1 * torch.sigmoid(x1))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, epsilon: float = 1e-6) -> torch.Tensor:
    """model_hub/utils.py:14-18"""
    variance = torch.mean(torch.square(x), dim=-1, keepdim=True)
    return (x * torch.rsqrt(variance + epsilon)) * weight


def apply_rope(position_ids: torch.Tensor, q: torch.Tensor, k: torch.Tensor, head_dim: int, cos_sin_cache: torch.Tensor):
    """model_hub/utils.py:20-106: q [B, S, Hq*D], k [B, S, Hkv*D], position_ids [B, S]; the fp32 table promotes the
    products to fp32 and the result is stored in the activation dtype."""
    b, s = position_ids.shape
    half = head_dim // 2
    cos = cos_sin_cache[position_ids.flatten(), :half].reshape(b, s, 1, half)
    sin = cos_sin_cache[position_ids.flatten(), half:].reshape(b, s, 1, half)

    def rot(x):
        xh = x.reshape(b, s, -1, head_dim)
        x1, x2 = xh[..., :half], xh[..., half:]
        out = torch.empty_like(xh)
        out[..., :half] = x1 * cos - x2 * sin
        out[..., half:] = x1 * sin + x2 * cos
        return out.reshape(x.shape)

    return rot(q), rot(k)


class LayerWeights:
    """Plain container: wqkv, bqkv, wo, gate_up_proj, down_proj, input_ln, post_ln, eps."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


def layer_prefill(h: torch.Tensor, w: LayerWeights, cos_sin_cache, pos0: int, num_heads: int, num_kv_heads: int,
                  head_dim: int, attention_fn):
    """model_hub/LLM.py:40-86 for one sequence; ``attention_fn(q [B,N,Hq,D], k, v) -> [B,N,Hq*D]``.
    Returns (hidden_states, key_states, value_states)."""
    b, n, dim = h.shape
    x = rmsnorm(h, w.input_ln, w.eps)
    qkv = F.linear(x, w.wqkv, w.bqkv)
    kvw = num_kv_heads * head_dim
    q, k, v = qkv.split([dim, kvw, kvw], dim=-1)
    pos = (torch.arange(n) + pos0).unsqueeze(0).repeat(b, 1)
    q, k = apply_rope(pos, q, k, head_dim, cos_sin_cache)
    q = q.reshape(b, n, num_heads, head_dim)
    k = k.reshape(b, n, num_kv_heads, head_dim)
    v = v.reshape(b, n, num_kv_heads, head_dim)
    attn = attention_fn(q, k, v)
    h = h + F.linear(attn.reshape(b, n, dim), w.wo)
    residual = h.clone()
    h = F.linear(silu_and_mul(F.linear(rmsnorm(h, w.post_ln, w.eps), w.gate_up_proj)), w.down_proj)
    return h + residual, k, v


def layer_decode(h: torch.Tensor, w: LayerWeights, cos_sin_cache, pos0: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len: int, decode_fn):
    """model_hub/LLM.py:88-116: h [B,1,dim]; the new key/value are written at position kv_len of the caches
    [B, capacity, Hkv, D]; ``decode_fn(q [B,1,Hq,D], k [B,L,Hkv,D], v) -> [B,1,Hq,D]`` sees kv_len+1 keys."""
    b, one, dim = h.shape
    x = rmsnorm(h, w.input_ln, w.eps)
    qkv = F.linear(x, w.wqkv, w.bqkv)
    kvw = num_kv_heads * head_dim
    q, k, v = qkv.split([dim, kvw, kvw], dim=-1)
    pos = torch.full((b, 1), pos0, dtype=torch.int64)
    q, k = apply_rope(pos, q, k, head_dim, cos_sin_cache)
    k_cache[:, kv_len] = k.reshape(b, num_kv_heads, head_dim)
    v_cache[:, kv_len] = v.reshape(b, num_kv_heads, head_dim)
    attn = decode_fn(q.reshape(b, 1, num_heads, head_dim), k_cache[:, :kv_len + 1], v_cache[:, :kv_len + 1])
    h = h + F.linear(attn.reshape(b, 1, dim), w.wo)
    return h + F.linear(silu_and_mul(F.linear(rmsnorm(h, w.post_ln, w.eps), w.gate_up_proj)), w.down_proj)
