"""Small Zuretar configurations for the tests, random model folders for them, and "sharp" variants
whose constants and weights are changed so that a lost key, a chunk edge that is one token off or a
lost state shows in the logits."""
import copy
import json
import os

import numpy as np
import torch


def _delta(heads, kv_heads, dim, vdim, conv, mlp=None, weights_of=None):
    d = {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
         "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def _parallel(left, right, mlp=None, weights_of=None):
    d = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def _left(heads, kv_heads, dim, vdim, scale, chunk, rot_dims, base, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk},
            "rot": rot}


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


# A: every kind of layer and feed-forward, layers that use another's weights (of both kinds), a chunk
# that is no multiple of a page, a partial rotation with YaRN scaling, a layer without feed-forward,
# a convolution of two taps, one head
_A_DELTA = _delta(4, 2, 16, 24, 4, _dense(96))
_A_PAR = _parallel(_left(4, 2, 32, 16, 0.2, 24, 16, 10000.0, (8.0, 64, 4.0, 1.0)), _right(2, 24, 40, (0.9, 0.99)),
                   _moe(8, 2, 40, (4, 2)))
ZUR_A = {"architecture": "Zuretar", "vocab": 300, "width": 64, "norm": {"eps": 1e-6}, "layers": [
    _A_DELTA, _A_PAR, dict(_A_DELTA, weights_of=0), _delta(1, 1, 40, 8, 2, None), dict(_A_PAR, weights_of=1),
    _delta(2, 1, 8, 8, 3, _moe(6, 3, 24))]}
# B: sizes the tensor-core products take; key and value sizes equal; a chunk of several pages; no
# scaling of the rotation; one expert chosen; a key size that takes eight lanes a column
_B_PAR = _parallel(_left(2, 1, 64, 64, 0.125, 128, 64, 500000.0), _right(3, 64, 32, (0.5, 0.95, 0.999)), _dense(144))
ZUR_B = {"architecture": "Zuretar", "vocab": 257, "width": 72, "norm": {"eps": 1e-5}, "layers": [
    _B_PAR, _delta(2, 2, 128, 64, 3, _moe(6, 1, 64)), _delta(2, 1, 256, 16, 4, _dense(80)), dict(_B_PAR, weights_of=0)]}
# C: sizes that no vector load and no tensor-core tile fits; a convolution of one tap; all experts
# chosen; groups that are all kept
ZUR_C = {"architecture": "Zuretar", "vocab": 101, "width": 50, "norm": {"eps": 1e-5}, "layers": [
    _delta(3, 1, 7, 5, 1, _moe(5, 5, 11)),
    _parallel(_left(3, 3, 10, 6, 0.4, 5, 6, 100.0, (2.0, 16, 3.0, 0.5)), _right(1, 9, 3, (0.8,)), _moe(6, 2, 9, (3, 3))),
    _delta(6, 3, 33, 35, 5, _dense(70))]}
ZUR = {"A": ZUR_A, "B": ZUR_B, "C": ZUR_C}
PAGE = {"A": 16, "B": 16, "C": 8}


def make_dir(tmp, name, store_dtype="float32", seed=None):
    from sglang_c_b200.config import resolve_architecture
    from sglang_c_b200.weights import write_random_model
    d = ZUR[name]
    arch = resolve_architecture(d)
    out = os.path.join(str(tmp), f"zur_{name}_{store_dtype}")
    if not os.path.exists(os.path.join(out, "model.safetensors")):
        write_random_model(out, arch, arch.config_class.from_dict(d), seed if seed is not None else 500 + ord(name),
                           scheme="varied", store_dtype=store_dtype)
    return out


def make_sharp_dir(tmp, name, store_dtype="float32"):
    """The model `name` with attention scores 16 times as large (queries and keys have unit root mean
    square whatever the weights are, so the config's multiplier is what sharpens the softmax: a key
    lost, misplaced, read from a stale page or let in across a chunk's edge then moves the logits by far
    more than rounding), the delta rule's decay close to one (A_log lowered: the state remembers
    hundreds of tokens), the linear attention's decays raised to 0.999 and more, and router corrections
    spread out (the choice differs from the order of the weights; choice scores go negative)."""
    import plain_zuretar
    from sglang_c_b200.weights.safetensors_io import write_safetensors
    base = make_dir(tmp, name, "float32")
    out = os.path.join(str(tmp), f"zur_sharp_{name}_{store_dtype}")
    if os.path.exists(os.path.join(out, "model.safetensors")):
        return out
    cfg, w = plain_zuretar.read_model_dir(base)
    cfg = copy.deepcopy(cfg)
    for entry in cfg["layers"]:
        if entry["type"] == "parallel":
            entry["mixer"]["left"]["scale"] *= 16.0
            n = len(entry["mixer"]["right"]["decay"])
            entry["mixer"]["right"]["decay"] = [0.999 + 0.0009 * i / max(n - 1, 1) for i in range(n)]
    tensors = {}
    rng = np.random.default_rng(77)
    for k, v in w.items():
        a = np.array(v, dtype=np.float32)
        if k.endswith(".mix.A_log"):
            a = a - 5.0
        elif k.endswith(".mlp.correction"):
            a = (rng.standard_normal(a.shape) * 0.8 - 0.6).astype(np.float32)
        t = torch.from_numpy(a)
        tensors[k] = t.to(torch.bfloat16) if (store_dtype == "bfloat16" and t.dim() >= 2) else t
    os.makedirs(out, exist_ok=True)
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(out, "model.safetensors"), tensors, metadata={"format": "pt"})
    return out
