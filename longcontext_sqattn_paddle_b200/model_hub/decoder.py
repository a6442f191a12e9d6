"""A random-weight decoder with the reference runtime's layer loops (model_hub/LLM.py:40-116, model_hub/qwen.py),
standing in for the checkpointed model as the CALLER of the attention operator: rmsnorm -> fused QKV projection
with bias -> rotary embedding (YaRN past 32768 positions) -> ``layer.prefill_attention`` / ``decode_attention``
-> output projection -> SwiGLU MLP in 8192-token chunks, layer by layer, with the KV cache of ``cache_hub``.

Matrix products are torch (cuBLAS) calls; rmsnorm, the rotation and SiLU*up are the library's row kernels; the
attention calls go through the same ``process_model`` / ``mp_triton_wrapper`` installation as in the reference.
With ``seq_shard=(rank, world)`` every rank runs the layer loop on its own token rows (equal contiguous shards, or
with ``shard_layout="zigzag"`` chunks r and 2G-1-r of 2G, which balances the dense causal layers) and the attention
operators are the sequence-parallel ones (``dist.sp_prefill_wrapper`` / ``dist.sp_dense_wrapper``); the KV cache
then holds the rank's keys, which is the layout of the cross-GPU split-KV decode (``dist.sp_decode``).
"""
from __future__ import annotations

import math
import types
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .. import ops
from ..cache_hub import flash_attn_cache
from ..sqattn import kernels as K


@dataclass
class DecoderConfig:
    num_hidden_layers: int = 28
    hidden_size: int = 3584
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    intermediate_size: int = 18944
    vocab_size: int = 152064
    rope_theta: float = 1000000.0
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 32768
    eos_token_id: int = 151645
    model_size_b: int = 7  # parameter count in billions, used by the cache's memory model

    @classmethod
    def qwen2_5_7b(cls, **overrides) -> "DecoderConfig":
        """The geometry of the reference's Qwen2.5-7B-Instruct configuration."""
        return cls(**overrides)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


def yarn_cos_sin_cache(head_dim: int, base: float, max_length: int, max_position_embeddings: int,
                       yarn_factor: float = 4.0, device="cpu") -> Tuple[torch.Tensor, float]:
    """cos|sin table [max_length, head_dim] in fp32 and the attention scaling already folded into it
    (model_hub/qwen.py:133-197): plain RoPE up to 32768 positions, YaRN (factor 4, beta_fast 32, beta_slow 1,
    scaling 0.1*ln(factor)+1) beyond."""
    idx = torch.arange(0, head_dim, 2, dtype=torch.float32)
    pos_freqs = base ** (idx / head_dim)
    inv_freq = 1.0 / pos_freqs
    scaling = 1.0
    if max_length > 32768:
        def correction_dim(num_rotations):
            return head_dim * math.log(max_position_embeddings / (num_rotations * 2 * math.pi)) / (2 * math.log(base))

        low = max(math.floor(correction_dim(32)), 0)
        high = min(math.ceil(correction_dim(1)), head_dim - 1)
        if low == high:
            high += 0.001
        ramp = torch.clamp((torch.arange(head_dim // 2, dtype=torch.float32) - low) / (high - low), 0, 1)
        extrapolation_factor = 1 - ramp
        inv_freq = (1.0 / (yarn_factor * pos_freqs)) * (1 - extrapolation_factor) + inv_freq * extrapolation_factor
        scaling = 0.1 * math.log(yarn_factor) + 1.0
    t = torch.arange(max_length, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq)
    table = torch.cat((freqs.cos() * scaling, freqs.sin() * scaling), dim=-1).contiguous()
    return table.to(device), scaling


class DecoderLayer:
    """Weights and attention hooks of one layer (model_hub/qwen.py:15-108): ``wqkv [Hq*D+2*Hkv*D, hidden]``,
    ``bqkv``, ``wo``, ``gate_up_proj [2*inter, hidden]``, ``down_proj``, the two norm weights and epsilons."""

    def __init__(self, layer_idx: int, config: DecoderConfig, dtype, device, attn_type: str, generator):
        c = config
        self.layer_idx, self.config, self.attention_type, self.device = layer_idx, c, attn_type, device
        self.num_layers, self.num_heads, self.num_key_value_heads = c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.hidden_size, self.head_dim = c.hidden_size, c.head_dim
        kv = c.num_key_value_heads * c.head_dim

        def w(*shape, std=0.02):
            return (torch.randn(*shape, generator=generator, device=device, dtype=torch.float32) * std).to(dtype)

        self.wqkv = w(c.hidden_size + 2 * kv, c.hidden_size)
        self.bqkv = w(c.hidden_size + 2 * kv, std=0.1)
        self.wo = w(c.hidden_size, c.hidden_size)
        self.gate_up_proj = w(2 * c.intermediate_size, c.hidden_size)
        self.down_proj = w(c.hidden_size, c.intermediate_size)
        self.input_layernorm_weight = torch.ones(c.hidden_size, dtype=dtype, device=device)
        self.post_attention_layernorm_weight = torch.ones(c.hidden_size, dtype=dtype, device=device)
        self.input_layernorm_variance_epsilon = c.rms_norm_eps
        self.post_attention_layernorm_variance_epsilon = c.rms_norm_eps

    def prefill_attention(self, query_states, key_states, value_states, layer_idx=None):
        """Dense causal attention [B,N,Hq,D] -> [B,N,Hq*D] (the un-replaced default, model_hub/qwen.py:38-48)."""
        if self.attention_type not in ("SQAttn", "SDPA", "FlashAttn"):
            raise ValueError(f"Unsupported attention type: {self.attention_type}")
        b, n, hq, d = query_states.shape
        out = K.attn_causal(query_states, key_states, value_states, tensor_layout="NHD", output_dtype=query_states.dtype)
        return out.reshape(b, n, hq * d)

    def decode_attention(self, query_states, key_states, value_states, layer_idx=None, kv_lens=None,
                         kv_lens_device=None):
        """One query token per sequence against the layer's cache [B,capacity,Hkv,D] (model_hub/qwen.py:50-56);
        ``kv_lens`` are the valid lengths (the reference attends to the whole allocation), on the host or, for a
        captured step, on the device."""
        if self.attention_type not in ("SQAttn", "SDPA", "FlashAttn"):
            raise ValueError(f"Unsupported attention type: {self.attention_type}")
        return ops.decode(query_states, key_states, value_states, layout="NHD", out_dtype=query_states.dtype,
                          kv_lens=kv_lens, kv_lens_device=kv_lens_device)


class RandomInitDecoder:
    """``LLM`` + ``QwenModel`` of the reference with seeded random weights (no checkpoint, no tokenizer)."""

    def __init__(self, config: DecoderConfig, max_length: int, dtype=torch.bfloat16, device="cuda:0",
                 attention_type: str = "SQAttn", seed: int = 0, seq_shard: Tuple[int, int] = (0, 1),
                 with_lm_head: bool = True, shard_layout: str = "contiguous"):
        self.config, self.max_length, self.dtype, self.attention_type = config, max_length, dtype, attention_type
        self.device = torch.device(device)
        self.device_map = str(device)
        c = config
        self.num_layers, self.num_heads, self.num_key_value_heads = c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.hidden_size, self.head_dim, self.vocab_size = c.hidden_size, c.head_dim, c.vocab_size
        self.base, self.max_position_embeddings, self.yarn_factor = c.rope_theta, c.max_position_embeddings, 4
        self.eos_tokens = [c.eos_token_id]
        self.num_gpus = 1
        self.rank, self.world = seq_shard
        self.shard_layout = shard_layout
        self.capture_layer_inps = None
        self.layer_mapping = {str(i): self.device_map for i in range(self.num_layers)}
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        self.embed_tokens = (torch.randn(c.vocab_size, c.hidden_size, generator=g, device=self.device) * 0.02).to(dtype)
        self.lm_head = ((torch.randn(c.vocab_size, c.hidden_size, generator=g, device=self.device) * 0.02).to(dtype)
                        if with_lm_head else self.embed_tokens)
        self.norm_weight = torch.ones(c.hidden_size, dtype=dtype, device=self.device)
        self.norm_variance_epsilon = c.rms_norm_eps
        self.cos_sin_cache, self.attention_scaling = yarn_cos_sin_cache(
            self.head_dim, self.base, max_length, self.max_position_embeddings, self.yarn_factor, self.device)
        self.layers = [DecoderLayer(i, c, dtype, self.device, attention_type, g) for i in range(self.num_layers)]
        self.kv_cache: Optional[flash_attn_cache] = None

    # ---- pieces of a layer (model_hub/qwen.py:292-379) -------------------------------------------------
    def word_embedding(self, inputs_id):
        return F.embedding(inputs_id, self.embed_tokens)

    def lm(self, hidden_states):
        return F.linear(hidden_states, self.lm_head).float()

    def layernorm(self, hidden_states, epsilon, weight, out=None):
        return ops.rmsnorm(hidden_states, weight, epsilon, out=out)

    def wqkv(self, hidden_states, layer):
        """Fused projection; returns the three column blocks as VIEWS of one [B,N,Hq*D+2*Hkv*D] buffer."""
        qkv = F.linear(hidden_states, layer.wqkv, layer.bqkv)
        kv = self.hidden_size // self.num_key_value_groups
        q, k, v = qkv.split([self.hidden_size, kv, kv], dim=-1)
        return qkv, q, k, v

    def position_embedd(self, qkv, seq_len, shard_offset=0, pos_device=None):
        """Rotate the query and key heads of the fused buffer in place at positions context + shard_offset + t
        (the context read from ``pos_device`` when a captured step is replayed)."""
        b = qkv.shape[0]
        pos0 = shard_offset if pos_device is not None else self.kv_cache.context + shard_offset
        ops.rope_qk(qkv.view(b * seq_len, qkv.shape[-1]), seq_len, self.num_heads + self.num_key_value_heads,
                    self.head_dim, self.cos_sin_cache, pos0, pos_device=pos_device)

    def wo(self, hidden_states, layer, bsz, seq_len, dim):
        return F.linear(hidden_states.reshape(bsz, seq_len, dim), layer.wo)

    def mlp(self, hidden_states, layer):
        return F.linear(ops.silu_mul(F.linear(hidden_states, layer.gate_up_proj)), layer.down_proj)

    # ---- layer loops (model_hub/LLM.py:40-116) ---------------------------------------------------------
    def layer_prefill(self, layer_idx, start_bdx, hidden_states):
        if self.capture_layer_inps is not None:
            self.capture_layer_inps.append(hidden_states.detach())
        bsz, seq_len, dim = hidden_states.shape
        layer = self.layers[layer_idx]
        normed = self.layernorm(hidden_states, layer.input_layernorm_variance_epsilon, layer.input_layernorm_weight)
        qkv, q, k, v = self.wqkv(normed, layer)
        del normed
        if self.world > 1:
            # every row range of this rank's shard is rotated at its own positions in the whole sequence
            from ..dist import ShardLayout
            lay = getattr(ShardLayout, self.shard_layout)(seq_len * self.world, self.world)
            base = 0
            for lo, hi in lay.segments(self.rank):
                self.position_embedd(qkv[:, base:base + hi - lo], hi - lo, shard_offset=lo)
                base += hi - lo
        else:
            self.position_embedd(qkv, seq_len)
        query_states = q.view(bsz, seq_len, self.num_heads, self.head_dim)
        key_states = k.view(bsz, seq_len, self.num_key_value_heads, self.head_dim)
        value_states = v.view(bsz, seq_len, self.num_key_value_heads, self.head_dim)
        key_states, value_states = self.kv_cache.prefill_update_kv_cache(query_states, key_states, value_states,
                                                                         layer_idx, start_bdx)
        attn_out = layer.prefill_attention(query_states, key_states, value_states, None)
        self.kv_cache.sync(layer_idx, start_bdx)
        hidden_states += self.wo(attn_out, layer, bsz, seq_len, dim)
        del qkv, q, k, v, query_states, key_states, value_states, attn_out
        step = max(1, 8192 // bsz)
        for s in range(0, seq_len, step):
            chunk = hidden_states[:, s:min(seq_len, s + step), :]
            normed = self.layernorm(chunk, layer.post_attention_layernorm_variance_epsilon,
                                    layer.post_attention_layernorm_weight)
            chunk += self.mlp(normed, layer)
        return hidden_states

    def layer_decode(self, layer_idx, hidden_states, dev=None):
        """``dev`` = (position int64 [1], lengths int32 [B]) on the GPU when the step is being captured for replay."""
        residual = hidden_states
        bsz, seq_len, dim = hidden_states.shape
        layer = self.layers[layer_idx]
        normed = self.layernorm(hidden_states, layer.input_layernorm_variance_epsilon, layer.input_layernorm_weight)
        qkv, q, k, v = self.wqkv(normed, layer)
        self.position_embedd(qkv, seq_len, pos_device=None if dev is None else dev[0])
        query_states = q.view(bsz, seq_len, self.num_heads, self.head_dim)
        key_states = k.view(bsz, seq_len, self.num_key_value_heads, self.head_dim)
        value_states = v.view(bsz, seq_len, self.num_key_value_heads, self.head_dim)
        lens = None if dev is not None else [x + 1 for x in self.kv_cache.valid_length_host]
        key_states, value_states = self.kv_cache.decode_update_kv_cache(key_states, value_states, layer_idx)
        attn_out = layer.decode_attention(query_states, key_states, value_states, None, kv_lens=lens,
                                          kv_lens_device=None if dev is None else dev[1])
        hidden_states = residual + self.wo(attn_out, layer, bsz, seq_len, dim)
        residual = hidden_states
        normed = self.layernorm(hidden_states, layer.post_attention_layernorm_variance_epsilon,
                                layer.post_attention_layernorm_weight)
        return residual + self.mlp(normed, layer)

    def prefill_forward(self, inputs_ids):
        """inputs_ids [B, N] (this rank's token rows when sharded) -> logits [B, 1, vocab] of the last position
        (when sharded: meaningful on the rank that owns the last token, the last rank for contiguous shards and
        rank 0 for the zig-zag layout; its last local row is the last token in both)."""
        bsz, _ = inputs_ids.shape
        last_hidden_states = torch.empty(bsz, 1, self.hidden_size, dtype=self.dtype, device=self.device)
        for start_bdx in range(bsz):
            hidden_states = self.word_embedding(inputs_ids[start_bdx:start_bdx + 1])
            for ldx in range(self.num_layers):
                hidden_states = self.layer_prefill(ldx, start_bdx, hidden_states)
            last_hidden_states[start_bdx:start_bdx + 1] = hidden_states[:, -1:, :]
        last_hidden_states = self.layernorm(last_hidden_states.contiguous(), self.norm_variance_epsilon, self.norm_weight)
        return self.lm(last_hidden_states)

    def decode_forward(self, inputs_ids, dev=None):
        hidden_states = self.word_embedding(inputs_ids)
        for ldx in range(self.num_layers):
            hidden_states = self.layer_decode(ldx, hidden_states, dev)
        hidden_states = self.layernorm(hidden_states[:, -1:, :].contiguous(), self.norm_variance_epsilon, self.norm_weight)
        return self.lm(hidden_states)

    # ---- one decode step as a replayable CUDA graph ---------------------------------------------------
    def _host_state(self):
        kc = self.kv_cache
        return kc.context, list(kc.valid_length_host)

    def _set_host_state(self, st):
        self.kv_cache.context, self.kv_cache.valid_length_host = st[0], list(st[1])

    def capture_decode_step(self, batch_size: int):
        """Capture ``decode_forward`` for replay: everything that changes from token to token (position, cache
        lengths, the index the new key/value rows go to) lives on the GPU and is advanced inside the graph, so
        ``decode_forward_graph`` is one graph launch per token with no host work between the layers."""
        kc = self.kv_cache
        if kc is None or kc.valid_length is None or not kc.allocated:
            raise RuntimeError("capture_decode_step needs a prefilled, GPU-resident cache")
        dev = self.device
        self._g_ids = torch.zeros(batch_size, 1, dtype=torch.int64, device=dev)
        self._g_pos = torch.full((1,), kc.context, dtype=torch.int64, device=dev)
        self._g_lens = torch.zeros(batch_size, dtype=torch.int32, device=dev)

        def step():
            self._g_lens.copy_((kc.valid_length + 1).to(torch.int32))
            logits = self.decode_forward(self._g_ids, dev=(self._g_pos, self._g_lens))   # advances valid_length
            self._g_pos += 1
            return logits

        # warm-up outside capture (library workspaces, lazy initialisation), then put the state back: the rows it
        # wrote at index valid_length are overwritten by the first real step
        host, vl = self._host_state(), kc.valid_length.clone()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        kc.valid_length.copy_(vl)
        self._g_pos.fill_(host[0])
        self._set_host_state(host)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._g_logits = step()
        self._set_host_state(host)   # capture ran the Python bookkeeping once without running any kernel

    def decode_forward_graph(self, inputs_ids):
        """``decode_forward`` through the captured graph; returns a view of the graph's logits buffer."""
        self._g_ids.copy_(inputs_ids)
        self._graph.replay()
        kc = self.kv_cache
        kc.context += 1
        kc.valid_length_host = [x + 1 for x in kc.valid_length_host]
        return self._g_logits

    # ---- generation (model_hub/LLM.py:160-235, model_hub/qwen.py:269-290) ------------------------------
    def init_kv_cache(self, real_input_length, valid_start):
        self.kv_cache = flash_attn_cache(
            valid_start=valid_start, layer_num=self.num_layers, batch_size=self.batch_size,
            max_length=self.max_new_length + real_input_length, num_key_value_heads=self.num_key_value_heads,
            num_heads=self.num_heads, head_dim=self.head_dim, dtype=self.dtype, layer_mapping=self.layer_mapping,
            num_gpus=self.num_gpus, model_size=self.config.model_size_b, device=self.device)

    def move(self):
        self.kv_cache.move_gpu()

    def inference(self, inputs_ids):
        outputs_ids = []
        logits = self.prefill_forward(inputs_ids=inputs_ids)
        output_ids = logits.argmax(dim=-1)
        outputs_ids.append(output_ids)
        self.move()
        for _ in range(self.max_new_length - 1):
            logits = self.decode_forward(inputs_ids=output_ids)
            output_ids = logits.argmax(dim=-1)
            outputs_ids.append(output_ids)
        return torch.cat(outputs_ids, dim=-1).tolist()

    def generate(self, attention_type, inputs_ids, attention_masks, max_new_length):
        bs, input_length = inputs_ids.shape
        assert input_length + max_new_length <= self.max_length, (
            f"Error: input_length({input_length}) + max_new_length({max_new_length}) exceeds max_length({self.max_length})")
        self.batch_size, self.input_length, self.max_new_length = bs, input_length, max_new_length
        self.attention_type = attention_type
        if attention_masks is None:
            valid_start = (0,) * bs
        else:
            valid_start = tuple(int(x) for x in (attention_masks.shape[1] - attention_masks.sum(dim=1)).tolist())
        self.init_kv_cache(input_length, valid_start)
        return self.inference(inputs_ids)


def install_sequence_parallel(model: RandomInitDecoder, window_sizes, args, group=None, p_fp8_mode: int = 0):
    """``process_model`` for a sharded model: every layer listed in ``window_sizes`` gets the sequence-parallel
    windowed operator (dist.sp_prefill_wrapper: all-reduce of the key sums, halo exchange of the prepared K/V rows),
    every other layer the sequence-parallel dense causal one (dist.sp_dense_wrapper: all-gather of K and V), both
    on the model's shard layout."""
    from ..dist import sp_dense_wrapper, sp_prefill_wrapper
    for i, layer in enumerate(model.layers):
        if i in window_sizes:
            fn = sp_prefill_wrapper(window_sizes[i]["bit8"], window_sizes[i]["bit4"], 256, args, group=group,
                                    p_fp8_mode=p_fp8_mode, layout=model.shard_layout)
        else:
            fn = sp_dense_wrapper(group=group, layout=model.shard_layout)
        layer.prefill_attention = types.MethodType(fn, layer)
    return model
