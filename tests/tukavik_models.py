"""Small Tukavik configurations for the tests, random model folders for them, and "sharp" variants
whose weights are changed so that a lost key or a lost state shows in the logits."""
import json
import os

import numpy as np
import torch


def _attn(kind, heads, dim, vdim, kv_rank, scale, ff=None, q_rank=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if q_rank is not None:
        m["q_rank"] = q_rank
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": kind, "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _gru(width, ff=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# A: every kind of layer, a shared latent, one head, sizes that are no powers of two
TUK_A = {"architecture": "Tukavik", "vocab": 300, "width": 64, "norm": {"eps": 1e-6}, "layers": [
    _attn("latent_attention", 2, 16, 24, 32, 0.25, ff=96),
    _gru(80, ff=72),
    _attn("latent_attention_2", 3, 8, 8, 40, 0.3, q_rank=24),
    _attn("latent_attention_2", 1, 20, 12, 40, 0.2, ff=64, q_rank=16, kv_from=2),
    _gru(128)]}
# B: latent sizes the tensor-core attention takes (64 and 128), a recurrence first, a layer that
# reads the latents of a layer of the other attention kind, a recurrence wider than one block
TUK_B = {"architecture": "Tukavik", "vocab": 257, "width": 72, "norm": {"eps": 1e-5}, "layers": [
    _gru(200),
    _attn("latent_attention", 4, 32, 32, 64, 0.18, ff=144),
    _attn("latent_attention_2", 2, 24, 40, 64, 0.2, q_rank=32, kv_from=1),
    _attn("latent_attention_2", 2, 64, 16, 128, 0.125, ff=80, q_rank=48),
    _gru(64, ff=100)]}
# C: sizes that no vector load and no tensor-core tile fits
TUK_C = {"architecture": "Tukavik", "vocab": 101, "width": 50, "norm": {"eps": 1e-5}, "layers": [
    _attn("latent_attention_2", 5, 6, 10, 20, 0.4, ff=70, q_rank=12),
    _gru(33),
    _attn("latent_attention", 1, 7, 3, 9, 0.37)]}
TUK = {"A": TUK_A, "B": TUK_B, "C": TUK_C}
PAGE = {"A": 16, "B": 16, "C": 8}


def make_dir(tmp, name, store_dtype="float32", seed=None):
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    d = TUK[name]
    arch = resolve_architecture(d)
    out = os.path.join(str(tmp), f"tuk_{name}_{store_dtype}")
    if not os.path.exists(os.path.join(out, "model.safetensors")):
        write_random_model(out, arch, arch.config_class.from_dict(d), seed if seed is not None else 300 + ord(name),
                           scheme="varied", store_dtype=store_dtype)
    return out


def make_sharp_dir(tmp, name, store_dtype="float32", factor=10.0, gate_shift=-3.0):
    """The model `name` with every query-side and key-side up-projection times `factor` (scores grow
    by its square: the softmax singles keys out, so a key lost, misplaced or read from a stale page
    moves the logits by far more than rounding), and every recurrence's gate bias shifted down (the
    gate opens to a few percent: the state remembers hundreds of tokens, so a state lost or reset at
    a cut shows long after)."""
    import plain_tukavik
    from sglang_c_b200.weights.safetensors_io import write_safetensors
    base = make_dir(tmp, name, "float32")
    out = os.path.join(str(tmp), f"tuk_sharp_{name}_{store_dtype}")
    if os.path.exists(os.path.join(out, "model.safetensors")):
        return out
    cfg, w = plain_tukavik.read_model_dir(base)
    tensors = {}
    for k, v in w.items():
        a = np.array(v, dtype=np.float32)
        if k.endswith((".mix.q", ".mix.uq", ".mix.uk")):
            a = a * factor
        elif k.endswith(".mix.z.b"):
            a = a + gate_shift
        t = torch.from_numpy(a)
        tensors[k] = t.to(torch.bfloat16) if (store_dtype == "bfloat16" and t.dim() >= 2) else t
    os.makedirs(out, exist_ok=True)
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(out, "model.safetensors"), tensors)
    return out
