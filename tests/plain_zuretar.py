"""A plain, slow restatement of the Zuretar architecture in float64 numpy, one function per
mechanism, sharing nothing with the engine: the oracle of the tests.  It reads a model folder
with its own small safetensors reader and runs whole sequences token by token where a
mechanism is a recurrence; there is no cache and no batch.

Notation: x [n, E] is the residual stream of n consecutive tokens from position 0; W x is
written x @ W.T for matrices stored [out, in].
"""
import json
import math
import os
import struct

import numpy as np


# -- files ---------------------------------------------------------------------------------
def read_model_dir(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    w = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = data[lo:hi]
        if meta["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif meta["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        elif meta["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        w[name] = a.astype(np.float64).reshape(meta["shape"])
    return cfg, w


# -- small functions -----------------------------------------------------------------------
def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def softplus(v):
    return np.maximum(v, 0.0) + np.log1p(np.exp(-np.abs(v)))


def silu(v):
    return v * sigmoid(v)


def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain, eps inside the root; gain None: no gain."""
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return y if gain is None else y * gain


# -- rotary positions with YaRN ------------------------------------------------------------
def yarn_frequencies(dims, base, scaling):
    """(frequency per pair [dims/2], multiplier of cos and sin).  Plain frequencies
    base^(-2i/dims); with scaling {factor, original, fast, slow} a pair's frequency is blended
    between itself and itself / factor by a ramp over the pair index."""
    half = dims // 2
    i = np.arange(half, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v, positions, dims, base, scaling):
    """v [n, heads, dim]: the first `dims` entries of every head are turned, entry i with entry
    i + dims/2; the rest pass."""
    f, mult = yarn_frequencies(dims, base, scaling)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * mult)[:, None, :], (np.sin(ang) * mult)[:, None, :]
    half = dims // 2
    a, b = v[..., :half], v[..., half:dims]
    out = v.copy()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# -- mixers ----------------------------------------------------------------------------------
def short_conv(x, taps):
    """Causal convolution over time per channel: x [n, C], taps [C, K], the last tap is the
    current token's; zeros before the start."""
    n, C = x.shape
    K = taps.shape[1]
    pad = np.concatenate([np.zeros((K - 1, C)), x], 0)
    out = np.zeros_like(x)
    for j in range(K):
        out += pad[j:j + n] * taps[:, j][None, :]
    return out


def gated_delta_mixer(h, w, p, m, eps):
    """The gated delta rule.  m: {heads, kv_heads, dim, vdim, conv}."""
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(n, G, D)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(n, G, D)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(n, H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)                                         # [n, H]
    decay = np.exp(-np.exp(w[p + "A_log"])[None, :] * softplus(h @ w[p + "a"].T + w[p + "dt_bias"][None, :]))
    gate = silu(h @ w[p + "g"].T).reshape(n, H, V)
    o = np.zeros((n, H, V))
    for hd in range(H):
        g = hd // (H // G)
        S = np.zeros((D, V))
        for t in range(n):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
    o = rms_norm(o, w[p + "norm"], eps) * gate
    return o.reshape(n, H * V) @ w[p + "o"].T


def chunked_sink_attention(h, w, p, m, eps):
    """Softmax attention with grouped key/value heads, rotary positions, unit-RMS queries and
    keys, a mask that lets position i see j <= i of its own chunk only, and a per-head sink in the
    denominator.  m: {heads, kv_heads, dim, vdim, rot, scale, mask}."""
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    pos = np.arange(n)
    q = rotate((h @ w[p + "q"].T).reshape(n, H, D), pos, rot["dims"], rot["base"], rot.get("scaling"))
    k = rotate((h @ w[p + "k"].T).reshape(n, G, D), pos, rot["dims"], rot["base"], rot.get("scaling"))
    v = (h @ w[p + "v"].T).reshape(n, G, V)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    size = m["mask"]["size"]
    out = np.zeros((n, H, V))
    for hd in range(H):
        g = hd // (H // G)
        for i in range(n):
            lo = (i // size) * size
            s = (k[lo:i + 1, g] @ q[i, hd]) * m["scale"]
            top = max(s.max(), w[p + "sink"][hd])
            e = np.exp(s - top)
            out[i, hd] = (e[:, None] * v[lo:i + 1, g]).sum(0) / (e.sum() + math.exp(w[p + "sink"][hd] - top))
    return out.reshape(n, H * V) @ w[p + "o"].T


def lightning_attention(h, w, p, m, eps):
    """Linear attention with a fixed decay per head: S <- decay S + k v^T, o = S^T q."""
    n = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(n, H, D)
    k = silu(h @ w[p + "k"].T).reshape(n, H, D)
    v = silu(h @ w[p + "v"].T).reshape(n, H, V)
    o = np.zeros((n, H, V))
    for hd in range(H):
        S = np.zeros((D, V))
        for t in range(n):
            S = m["decay"][hd] * S + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms_norm(o.reshape(n, H * V), w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def side_by_side_mixer(h, w, p, m, eps):
    left = chunked_sink_attention(h, w, p + "left.", m["left"], eps)
    right = lightning_attention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


# -- feed-forwards -----------------------------------------------------------------------------
def dense_ff(h, w, p):
    g = h @ w[p + "gate"].T + w[p + "gate.b"]
    u = h @ w[p + "up"].T + w[p + "up.b"]
    return (silu(g) * u) @ w[p + "down"].T + w[p + "down.b"]


def route(h, w, p, r):
    """(chosen experts [n, top], their weights [n, top]).  r: {experts, top, groups{count, keep}}."""
    n = h.shape[0]
    s = sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"][None, :]
    E, top = r["experts"], r["top"]
    groups = r.get("groups")
    if groups:
        per = E // groups["count"]
        gs = np.sort(choice.reshape(n, groups["count"], per), -1)[..., -2:].sum(-1)
        keep = np.argsort(-gs, -1, kind="stable")[:, :groups["keep"]]
        allowed = np.zeros((n, groups["count"]), dtype=bool)
        np.put_along_axis(allowed, keep, True, -1)
        choice = np.where(np.repeat(allowed, per, -1), choice, -np.inf)
    chosen = np.argsort(-choice, -1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, -1)


def moe_ff(h, w, p, mlp):
    chosen, weight = route(h, w, p, mlp["router"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t], weight[t]):
            pe = f"{p}e{e}."
            z = silu(w[pe + "gate"] @ h[t]) * (w[pe + "up"] @ h[t])
            out[t] += a * (w[pe + "down"] @ z)
    return out


# -- the model ---------------------------------------------------------------------------------
def layer(x, w, cfg, i):
    """x + mixer(norm(x)) + ff(norm(x)): one norm, both sublayers read it."""
    entry = cfg["layers"][i]
    src = entry.get("weights_of", i)
    p = f"l{src}."
    eps = cfg["norm"]["eps"]
    h = rms_norm(x, w[p + "norm1"], eps)
    if entry["type"] == "delta":
        y = gated_delta_mixer(h, w, p + "mix.", entry["mixer"], eps)
    elif entry["type"] == "parallel":
        y = side_by_side_mixer(h, w, p + "mix.", entry["mixer"], eps)
    else:
        raise ValueError(entry["type"])
    mlp = entry.get("mlp")
    if mlp is not None:
        y = y + (dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp))
    return x + y


def forward(cfg, w, tokens, streams=None):
    """Logits [n, vocab] of a whole sequence from position 0.  `streams`, a list, takes the
    residual stream after every layer."""
    x = w["embed"][np.asarray(tokens)]
    for i in range(len(cfg["layers"])):
        x = layer(x, w, cfg, i)
        if streams is not None:
            streams.append(x.copy())
    return rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T


def forward_dir(model_dir, tokens):
    cfg, w = read_model_dir(model_dir)
    return forward(cfg, w, tokens)
