"""A plain, slow restatement of the Tukavik architecture in float64 numpy, one function per
mechanism, sharing nothing with the engine: the oracle of the tests.  It reads a model folder
with its own small safetensors reader and runs whole sequences; there is no cache and no batch.

Notation: x [n, E] is the residual stream of n consecutive tokens from position 0.
"""
import json
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
    return np.log1p(np.exp(v))


def silu(v):
    return v * sigmoid(v)


def layer_norm(x, gain, eps):
    """Mean removed, divided by sqrt(variance + eps) with the variance the mean squared deviation,
    times a gain; no bias."""
    d = x - x.mean(-1, keepdims=True)
    return d / np.sqrt((d * d).mean(-1, keepdims=True) + eps) * gain


def rms_norm(x, gain, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * gain


def sinusoid(n, width, base=10000.0, first=0):
    """[n, width]: entry 2i of position p is sin(p * base^(-2i/width)), entry 2i+1 its cosine."""
    out = np.zeros((n, width))
    p = np.arange(first, first + n, dtype=np.float64)[:, None]
    i = np.arange((width + 1) // 2, dtype=np.float64)[None, :]
    ang = p * base ** (-2.0 * i / width)
    out[:, 0::2] = np.sin(ang)
    out[:, 1::2] = np.cos(ang)[:, :width // 2]
    return out


def xielu(z, p, q):
    pos = softplus(p) * z * z + z / 2
    neg = (0.5 + softplus(q)) * (np.expm1(z) - z) + z / 2
    return np.where(z > 0, pos, neg)


def min_gru(h, wz, bz, wx, bx, wg, wo, state=None):
    """(out [n, E], final state): the gates read the current token only."""
    z = sigmoid(h @ wz.T + bz)
    u = h @ wx.T + bx
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    s = np.zeros(wz.shape[0]) if state is None else state
    states = np.empty_like(z)
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        states[t] = s
    return (states * silu(h @ wg.T)) @ wo.T, s


def latent(h, w_down, gain, eps):
    """What an attention layer keeps per position."""
    return rms_norm(h @ w_down.T, gain, eps)


def latent_attention(q, c, w_uk, w_uv, w_o, heads, scale):
    """q [n, heads*dim]; c [n, rank] the latents of the same n positions; causal, ordinary softmax."""
    n = q.shape[0]
    dim, vdim = w_uk.shape[0] // heads, w_uv.shape[0] // heads
    k = (c @ w_uk.T).reshape(n, heads, dim)
    v = (c @ w_uv.T).reshape(n, heads, vdim)
    qh = q.reshape(n, heads, dim)
    out = np.zeros((n, heads, vdim))
    for i in range(n):
        s = np.einsum("hd,jhd->hj", qh[i], k[:i + 1]) * scale
        s = np.exp(s - s.max(-1, keepdims=True))
        a = s / s.sum(-1, keepdims=True)
        out[i] = np.einsum("hj,jhv->hv", a, v[:i + 1])
    return out.reshape(n, heads * vdim) @ w_o.T


def dense_ff(h, w_up, w_down, act):
    return xielu(h @ w_up.T, act[0], act[1]) @ w_down.T


def depth_average(streams, weights):
    return sum(weights[j] * streams[j] for j in range(len(streams)))


# -- the model -------------------------------------------------------------------------------
def forward(cfg, w, tokens, return_layers=False):
    """float64 logits [n, vocab] of the whole sequence."""
    E, eps = cfg["width"], cfg["norm"]["eps"]
    tokens = np.asarray(tokens)
    x = w["embed"][tokens] + sinusoid(len(tokens), E)
    streams, latents, after = [x], {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "mingru":
            y, _ = min_gru(h, w[p + "mix.z"], w[p + "mix.z.b"], w[p + "mix.x"], w[p + "mix.x.b"],
                           w[p + "mix.g"], w[p + "mix.o"])
        else:
            if layer["type"] == "latent_attention":
                q = h @ w[p + "mix.q"].T
            else:
                q = rms_norm(h @ w[p + "mix.dq"].T, w[p + "mix.dq.norm"], eps) @ w[p + "mix.uq"].T
            if "kv_from" in m and m["kv_from"] is not None:
                c = latents[m["kv_from"]]
            else:
                c = latent(h, w[p + "mix.dkv"], w[p + "mix.dkv.norm"], eps)
                latents[i] = c
            y = latent_attention(q, c, w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.o"], m["heads"], m["scale"])
        x = x + layer_norm(y, w[p + "norm1b"], eps)
        if layer["mlp"] is not None:
            h = layer_norm(x, w[p + "norm2"], eps)
            x = x + layer_norm(dense_ff(h, w[p + "mlp.up"], w[p + "mlp.down"], w[p + "mlp.act"]), w[p + "norm2b"], eps)
        streams.append(x)
        x = depth_average(streams, w[p + "dwa"])
        after.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, after) if return_layers else logits


def forward_dir(model_dir, tokens):
    cfg, w = read_model_dir(model_dir)
    return forward(cfg, w, tokens)
