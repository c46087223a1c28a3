"""The callers of the hot path, restated from ratchet-models so the benchmark configurations can be
scheduled through the lazy ``Tensor`` API exactly as the reference schedules them:

* Phi-3 decoder (crates/ratchet-models/src/phi3/{attn,mlp,model}.rs),
* the Phi-2 MLP block inside its parallel-residual layer (phi2/mlp.rs:13-15, phi2/model.rs:78-89),
* the Whisper encoder (whisper/{encoder,residual_block,mha,mlp}.rs).

They only call ``Tensor`` builder methods, as ``Module::schedule`` does in the reference; no device
code lives here.
"""
from __future__ import annotations

from typing import List, Optional

from . import capi
from .nn import KVCache, KVEntry, LayerNorm, Linear, RMSNorm, RotaryEmbedding, Embedding


# ---------------------------------------------------------------------------------------- Phi-3
class Phi3SelfAttention:
    """phi3/attn.rs:88-159."""

    def __init__(self, qkv: Linear, o: Linear, rope: RotaryEmbedding, n_heads: int, n_kv_heads: int, softmax_scale):
        self.qkv, self.o, self.rope = qkv, o, rope
        self.n_heads, self.n_kv_heads, self.softmax_scale = n_heads, n_kv_heads, softmax_scale

    def schedule(self, x, mask=None, cache: Optional[KVEntry] = None):
        batch, q_len, n_state = x.shape()
        hdim = n_state // self.n_heads
        kv_x_hdim = self.n_kv_heads * hdim
        qkv = self.qkv.schedule(x)
        return self.o.schedule(self.attend(qkv, batch, q_len, n_state, mask, cache))

    def attend(self, qkv, batch, q_len, n_state, mask=None, cache: Optional[KVEntry] = None):
        """Everything between the fused qkv projection and the output projection (attn.rs:95-157)."""
        hdim = n_state // self.n_heads
        kv_x_hdim = self.n_kv_heads * hdim
        query_pos = self.n_heads * hdim
        key_pos = query_pos + kv_x_hdim
        value_pos = key_pos + kv_x_hdim
        q = qkv.slice([(0, batch), (0, q_len), (0, query_pos)])
        k = qkv.slice([(0, batch), (0, q_len), (query_pos, key_pos)])
        v = qkv.slice([(0, batch), (0, q_len), (key_pos, value_pos)])
        q = q.view([batch, q_len, self.n_heads, hdim]).permute([0, 2, 1, 3])
        k = k.view([batch, q_len, self.n_kv_heads, hdim]).permute([0, 2, 1, 3])
        v = v.view([batch, q_len, self.n_kv_heads, hdim]).permute([0, 2, 1, 3])
        offset = cache.entries if cache is not None else 0
        q_dt = q.dt()
        q = self.rope.schedule(q.full(), offset).cast(q_dt)
        k = self.rope.schedule(k.full(), offset).cast(q_dt)
        if cache is not None:
            k = cache.k_cache.cache(k, 2, offset)
            v = cache.v_cache.cache(v, 2, offset)
        attn = q.full().matmul(k.full(), False, True).mul(self.softmax_scale).cast(q_dt)
        if mask is not None:
            attn = attn.add(mask.cast(attn.dt()))
        w = attn.full().softmax(3).cast(v.dt())
        wv = w.matmul(v, False, False).permute([0, 2, 1, 3])
        return wv.view([batch, q_len, n_state])


class Phi3MLP:
    """phi3/mlp.rs:31-39: fused gate_up projection, up * silu(gate), down projection."""

    def __init__(self, up_proj: Linear, down_proj: Linear):
        self.up_proj, self.down_proj = up_proj, down_proj

    def schedule(self, x):
        input_dt = x.dt()
        up_states = self.up_proj.schedule(x)
        a, b, c = up_states.shape()
        gate = up_states.slice([(0, a), (0, b), (0, c // 2)])
        up = up_states.slice([(0, a), (0, b), (c // 2, c)])
        up = up.mul(gate.full().silu().cast(input_dt))
        return self.down_proj.schedule(up)


class Phi3DecoderLayer:
    """phi3/model.rs:103-118."""

    def __init__(self, input_norm: RMSNorm, self_attn: Phi3SelfAttention, ffn_norm: RMSNorm, mlp: Phi3MLP):
        self.input_norm, self.self_attn, self.ffn_norm, self.mlp = input_norm, self_attn, ffn_norm, mlp

    def schedule(self, x, mask=None, cache: Optional[KVEntry] = None):
        residual = x
        xs = self.input_norm.schedule(x)
        attn_output = self.self_attn.schedule(xs, mask, cache)
        xs = residual.add(attn_output)
        residual = xs
        xs = self.ffn_norm.schedule(xs)
        xs = self.mlp.schedule(xs)
        return residual.add(xs)


class Phi3:
    """phi3/model.rs:134-156 (decode only: no mask is generated for seq_len <= 1, as there)."""

    def __init__(self, embedding: Embedding, layers: List[Phi3DecoderLayer], ln_post: RMSNorm, lm_head: Linear, kv_cache: KVCache):
        self.embedding, self.layers, self.ln_post, self.lm_head, self.kv_cache = embedding, layers, ln_post, lm_head, kv_cache

    def schedule(self, ids, mask=None):
        x = self.embedding.schedule(ids)
        _, seq_len, n_state = x.shape()
        for i, layer in enumerate(self.layers):
            x = layer.schedule(x, mask, self.kv_cache[i])
        x = self.ln_post.schedule(x)
        x = x.slice([(0, 1), (seq_len - 1, seq_len), (0, n_state)])
        return self.lm_head.schedule(x)


# ---------------------------------------------------------------------------------------- Phi-2
class Phi2MLPBlock:
    """LayerNorm -> fc1 -> gelu -> fc2 -> + x: the MLP arm of phi2/model.rs:78-89 with phi2/mlp.rs:13-15."""

    def __init__(self, ln: LayerNorm, fc1: Linear, fc2: Linear):
        self.ln, self.fc1, self.fc2 = ln, fc1, fc2

    def schedule(self, x):
        h = self.ln.schedule(x)
        return self.fc2.schedule(self.fc1.schedule(h).gelu()).add(x)


# ---------------------------------------------------------------------------------------- Whisper
class WhisperMHA:
    """whisper/mha.rs:57-127; ``dk`` is the [1] tensor holding head_dim^-0.25."""

    def __init__(self, q: Linear, k: Linear, v: Linear, o: Linear, n_heads: int, dk):
        self.q, self.k, self.v, self.o, self.n_heads, self.dk = q, k, v, o, n_heads, dk

    def schedule(self, x):
        q = self.q.schedule(x)
        k = self.k.schedule(x)
        v = self.v.schedule(x)
        bs, n_ctx, n_state = q.shape()
        q_dt = q.dt()
        hdim = n_state // self.n_heads
        q = q.view([bs, n_ctx, self.n_heads, hdim]).permute([0, 2, 1, 3]).mul(self.dk)
        k = k.view([bs, n_ctx, self.n_heads, hdim]).permute([0, 2, 3, 1]).mul(self.dk)
        v = v.view([bs, n_ctx, self.n_heads, hdim]).permute([0, 2, 1, 3])
        qk = q.matmul(k, False, False).full()
        w = qk.softmax(3).cast(q_dt)
        wv = w.matmul(v, False, False).permute([0, 2, 1, 3]).view([bs, n_ctx, n_state])
        return self.o.schedule(wv)


class WhisperMLP:
    """whisper/mlp.rs:18-22."""

    def __init__(self, l1: Linear, l2: Linear):
        self.l1, self.l2 = l1, l2

    def schedule(self, x):
        return self.l2.schedule(self.l1.schedule(x).full().gelu().cast(x.dt()))


class WhisperBlock:
    """whisper/residual_block.rs:30-51 without cross attention (encoder)."""

    def __init__(self, attn_ln: LayerNorm, attn: WhisperMHA, mlp_ln: LayerNorm, mlp: WhisperMLP):
        self.attn_ln, self.attn, self.mlp_ln, self.mlp = attn_ln, attn, mlp_ln, mlp

    def schedule(self, x):
        attn = x.add(self.attn.schedule(self.attn_ln.schedule(x)))
        return self.mlp.schedule(self.mlp_ln.schedule(attn)).add(attn)


class WhisperEncoder:
    """whisper/encoder.rs:49-55,108-122: conv stem in f32 (conv1d k3 s1 -> gelu -> conv1d k3 s2 -> gelu,
    permute, + positional embedding), cast to the activation dtype, blocks, final LayerNorm."""

    def __init__(self, conv1_w, conv1_b, conv2_w, conv2_b, pos_embed, blocks: List[WhisperBlock], ln_post: LayerNorm, activation_dt: int):
        self.conv1_w, self.conv1_b, self.conv2_w, self.conv2_b = conv1_w, conv1_b, conv2_w, conv2_b
        self.pos_embed, self.blocks, self.ln_post, self.activation_dt = pos_embed, blocks, ln_post, activation_dt

    def schedule(self, mel):
        x = mel.full().conv1d(self.conv1_w, self.conv1_b, 1, 1).gelu()
        x = x.conv1d(self.conv2_w, self.conv2_b, 2, 1).gelu()
        x = x.permute([0, 2, 1]).add(self.pos_embed.full())
        x = x.cast(self.activation_dt)
        for blk in self.blocks:
            x = blk.schedule(x)
        return self.ln_post.schedule(x)
