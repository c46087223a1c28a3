"""Seeded synthetic weights for the benchmark configurations and constructors that wrap them in either
tensor backend (CUDA ``Tensor`` or the oracle's ``OTensor``), so both run the same ``schedule()``.

Real checkpoints are not available offline; shapes and value distributions follow the configuration
descriptions (weights N(0, 0.02), norm scales 1, biases 0 unless stated).
"""
import numpy as np

from oracle import oracle as orc
from ratchet_b200 import callers, nn

F32, F16, Q8_0F, Q8_0H = 0, 1, 5, 6


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def _weight(g, shape, quant):
    """returns (raw, dt): float array, or Q8_0 buffer in ratchet's layout (quant.rs:51-99)."""
    w = (g.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
    if quant == "f32":
        return w, F32
    if quant == "f16":
        return w.astype(np.float16), F16
    if quant == "q8f":
        return orc.quantize_q8(w), Q8_0F
    if quant == "q8h":
        return orc.quantize_q8(w.astype(np.float16)), Q8_0H
    raise ValueError(quant)


def _wrap(T, dev, raw, dt, shape):
    if dt in (Q8_0F, Q8_0H):
        return T.from_quantized(raw, dt, shape, dev)
    return T.from_data(raw, device=dev)


# ------------------------------------------------------------------------------------- Phi-3
def phi3_weights(seed, n_layers, d=3072, n_heads=32, ffn=8192, vocab=32064, quant="q8h"):
    g = rng(seed)
    L = []
    for _ in range(n_layers):
        L.append({
            "attn_norm": np.ones(d, np.float32) + 0.1 * g.standard_normal(d).astype(np.float32),
            "qkv": _weight(g, (3 * d, d), quant), "o": _weight(g, (d, d), quant),
            "ffn_norm": np.ones(d, np.float32) + 0.1 * g.standard_normal(d).astype(np.float32),
            "up": _weight(g, (2 * ffn, d), quant), "down": _weight(g, (d, ffn), quant),
        })
    return {"layers": L, "embd": _weight(g, (vocab, d), quant), "ln_post": np.ones(d, np.float32),
            "lm_head": _weight(g, (vocab, d), quant), "d": d, "n_heads": n_heads, "ffn": ffn, "vocab": vocab}


def phi3_kv(W, kv_prior, act_np, max_cache=4096, kv_seed=5):
    """Per layer (k_cache, v_cache) [1, H, max_cache, hd], zero except `kv_prior` N(0,1) positions."""
    d, H = W["d"], W["n_heads"]
    hd = d // H
    g = rng(kv_seed)
    out = []
    for _ in W["layers"]:
        kc = np.zeros((1, H, max_cache, hd), act_np)
        vc = np.zeros((1, H, max_cache, hd), act_np)
        kc[:, :, :kv_prior] = g.standard_normal((1, H, kv_prior, hd)).astype(act_np)
        vc[:, :, :kv_prior] = g.standard_normal((1, H, kv_prior, hd)).astype(act_np)
        out.append((kc, vc))
    return out


def phi3_decoder(dev, W, kv_prior, max_cache=4096, kv_seed=5):
    """The fused decode engine over the same weights and caches as phi3_model (f16 activations)."""
    from ratchet_b200 import capi
    from ratchet_b200.decoder import Decoder, DecoderConfig, DecoderLayer
    d, H = W["d"], W["n_heads"]
    hd = d // H
    kv = phi3_kv(W, kv_prior, np.float16, max_cache, kv_seed)
    wdt = W["embd"][1]
    q = lambda rd, shape: dev.from_quantized(rd[0], rd[1], shape)
    layers = []
    for li, lw in enumerate(W["layers"]):
        layers.append(DecoderLayer(dev.from_numpy(lw["attn_norm"]), q(lw["qkv"], (3 * d, d)), q(lw["o"], (d, d)), dev.from_numpy(lw["ffn_norm"]),
                                   q(lw["up"], (2 * W["ffn"], d)), q(lw["down"], (d, W["ffn"])),
                                   dev.from_numpy(kv[li][0][0]), dev.from_numpy(kv[li][1][0])))
    cfg = DecoderConfig(len(layers), d, H, H, hd, W["ffn"], W["vocab"], max_cache, hd, 10000.0, 1e-5, wdt)
    dec = Decoder(dev, cfg, layers, q(W["embd"], (W["vocab"], d)), dev.from_numpy(W["ln_post"]), q(W["lm_head"], (W["vocab"], d)))
    dec.position = kv_prior
    return dec


def phi3_decoder_sharded(dev, W, kv_prior, comm, max_cache=4096, kv_seed=5):
    """The same engine with every Linear sharded over the ranks of `comm` (this rank's rows, its own KV heads)."""
    from ratchet_b200.comm import decoder_shard_ranges, take_rows_q8
    from ratchet_b200.decoder import Decoder, DecoderConfig, DecoderLayer
    d, H, ffn, vocab = W["d"], W["n_heads"], W["ffn"], W["vocab"]
    hd = d // H
    R = decoder_shard_ranges(H, H, hd, d, ffn, vocab, comm.rank, comm.world)
    kv = phi3_kv(W, kv_prior, np.float16, max_cache, kv_seed)
    wdt = W["embd"][1]
    rows = lambda rng_list: sum(b - a for a, b in rng_list)

    def shard(rd, n_rows, k, key):
        return dev.from_quantized(take_rows_q8(rd[0], rd[1], n_rows, k, R[key]), rd[1], (rows(R[key]), k))

    h0, h1 = R["kv_heads"]
    layers = []
    for li, lw in enumerate(W["layers"]):
        layers.append(DecoderLayer(dev.from_numpy(lw["attn_norm"]), shard(lw["qkv"], 3 * d, d, "qkv"), shard(lw["o"], d, d, "o"),
                                   dev.from_numpy(lw["ffn_norm"]), shard(lw["up"], 2 * ffn, d, "gate_up"), shard(lw["down"], d, ffn, "down"),
                                   dev.from_numpy(np.ascontiguousarray(kv[li][0][0, h0:h1])),
                                   dev.from_numpy(np.ascontiguousarray(kv[li][1][0, h0:h1]))))
    cfg = DecoderConfig(len(layers), d, H, H, hd, ffn, vocab, max_cache, hd, 10000.0, 1e-5, wdt)
    dec = Decoder(dev, cfg, layers, dev.from_quantized(W["embd"][0], wdt, (vocab, d)), dev.from_numpy(W["ln_post"]),
                  shard(W["lm_head"], vocab, d, "lm_head"), comm=comm)
    dec.position = kv_prior
    return dec


def phi3_model(T, dev, W, kv_prior, act_np, max_cache=4096, kv_seed=5):
    """Builds callers.Phi3 with a KV cache holding `kv_prior` N(0,1) positions (phi3/model.rs:160-202)."""
    d, H = W["d"], W["n_heads"]
    hd = d // H
    kv = phi3_kv(W, kv_prior, act_np, max_cache, kv_seed)
    scale = T.from_data(np.array([1.0 / np.sqrt(np.float32(hd))], np.float32), device=dev)
    layers, entries = [], []
    for li, lw in enumerate(W["layers"]):
        attn = callers.Phi3SelfAttention(nn.Linear(_wrap(T, dev, *lw["qkv"], (3 * d, d))), nn.Linear(_wrap(T, dev, *lw["o"], (d, d))),
                                         nn.RotaryEmbedding(hd, False, 10000.0, 1.0), H, H, scale)
        mlp = callers.Phi3MLP(nn.Linear(_wrap(T, dev, *lw["up"], (2 * W["ffn"], d))), nn.Linear(_wrap(T, dev, *lw["down"], (d, W["ffn"]))))
        layers.append(callers.Phi3DecoderLayer(nn.RMSNorm(T.from_data(lw["attn_norm"], device=dev), 1e-5), attn,
                                               nn.RMSNorm(T.from_data(lw["ffn_norm"], device=dev), 1e-5), mlp))
        kc, vc = kv[li]
        entries.append(nn.KVEntry(T.from_data(kc, device=dev), T.from_data(vc, device=dev), kv_prior))
    model = callers.Phi3(nn.Embedding(_wrap(T, dev, *W["embd"], (W["vocab"], d))), layers,
                         nn.RMSNorm(T.from_data(W["ln_post"], device=dev), 1e-5),
                         nn.Linear(_wrap(T, dev, *W["lm_head"], (W["vocab"], d))), nn.KVCache(entries))
    return model


# ------------------------------------------------------------------------------------- Phi-2 MLP block
def phi2_mlp_weights(seed, d=2560, ffn=10240):
    g = rng(seed)
    return {"x": g.standard_normal((1, 64, d)).astype(np.float32), "gamma": np.ones(d, np.float32), "beta": np.zeros(d, np.float32),
            "w1": _weight(g, (ffn, d), "f32")[0], "b1": np.zeros(ffn, np.float32),
            "w2": _weight(g, (d, ffn), "f32")[0], "b2": np.zeros(d, np.float32)}


def phi2_mlp_block(T, dev, W):
    t = lambda a: T.from_data(a, device=dev)
    return callers.Phi2MLPBlock(nn.LayerNorm(t(W["gamma"]), t(W["beta"]), 1e-5), nn.Linear(t(W["w1"]), t(W["b1"])),
                                nn.Linear(t(W["w2"]), t(W["b2"])))


# ------------------------------------------------------------------------------------- Whisper encoder
def sinusoids(length, channels, max_timescale=10000.0):
    inc = np.log(max_timescale) / (channels // 2 - 1)
    inv = np.exp(-inc * np.arange(channels // 2))
    t = np.arange(length)[:, None] * inv[None, :]
    return np.concatenate([np.sin(t), np.cos(t)], 1).astype(np.float32)


def whisper_weights(seed, n_mels=80, n_ctx=1500, d=384, n_heads=6, mlp=1536, n_layers=4, quant="f32"):
    g = rng(seed)
    W = {"conv1_w": _weight(g, (d, n_mels, 3), "f32")[0], "conv1_b": (g.standard_normal(d) * 0.02).astype(np.float32),
         "conv2_w": _weight(g, (d, d, 3), "f32")[0], "conv2_b": (g.standard_normal(d) * 0.02).astype(np.float32),
         "pos": sinusoids(n_ctx, d), "blocks": [], "ln_post": (np.ones(d, np.float32), np.zeros(d, np.float32)),
         "d": d, "n_heads": n_heads, "mlp": mlp, "n_ctx": n_ctx, "quant": quant}
    for _ in range(n_layers):
        b = {"attn_ln": (np.ones(d, np.float32), np.zeros(d, np.float32)), "mlp_ln": (np.ones(d, np.float32), np.zeros(d, np.float32))}
        for name, shape in (("q", (d, d)), ("k", (d, d)), ("v", (d, d)), ("o", (d, d)), ("fc1", (mlp, d)), ("fc2", (d, mlp))):
            b[name] = _weight(g, shape, quant)
            b[name + "_b"] = None if name == "k" else (g.standard_normal(shape[0]) * 0.02).astype(np.float32)   # k_proj has no bias
        W["blocks"].append(b)
    return W


def whisper_encoder(T, dev, W):
    t = lambda a: T.from_data(a, device=dev)
    d, H = W["d"], W["n_heads"]
    act = F16 if W["quant"] in ("f16", "q8h") else F32
    act_np = np.float16 if act == F16 else np.float32
    dk = t(np.array([np.float32(d // H) ** np.float32(-0.25)], np.float32).astype(act_np))
    blocks = []
    for b in W["blocks"]:
        lin = lambda n, shape: nn.Linear(_wrap(T, dev, *b[n], shape), None if b[n + "_b"] is None else t(b[n + "_b"]))
        mha = callers.WhisperMHA(lin("q", (d, d)), lin("k", (d, d)), lin("v", (d, d)), lin("o", (d, d)), H, dk)
        mlp = callers.WhisperMLP(lin("fc1", (W["mlp"], d)), lin("fc2", (d, W["mlp"])))
        blocks.append(callers.WhisperBlock(nn.LayerNorm(t(b["attn_ln"][0]), t(b["attn_ln"][1]), 1e-5), mha,
                                           nn.LayerNorm(t(b["mlp_ln"][0]), t(b["mlp_ln"][1]), 1e-5), mlp))
    return callers.WhisperEncoder(t(W["conv1_w"]), t(W["conv1_b"]), t(W["conv2_w"]), t(W["conv2_b"]), t(W["pos"]), blocks,
                                  nn.LayerNorm(t(W["ln_post"][0]), t(W["ln_post"][1]), 1e-5), act)
