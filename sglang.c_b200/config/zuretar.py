"""Typed configuration of the Zuretar architecture: a decoder whose config.json lists its layers
one by one.  A layer has one RMS norm that a mixer and a feed-forward both read; the mixer is a
gated delta rule ("delta") or softmax attention beside a linear attention ("parallel"); the
feed-forward is dense, a mixture of experts, or absent.  A layer may use the weights of an
earlier layer (`weights_of`) with a cache and state of its own.  Every size and every constant
that may differ between models comes from the file:

    {"architecture": "Zuretar", "vocab": V, "width": E, "norm": {"eps": e},
     "layers": [{"type": "delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                                    "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                           "right": {"heads", "dim", "vdim", "decay": [per head]}},
                 "mlp": {"kind": "moe", "expert": {"ff": F},
                         "router": {"experts", "top", "groups": {"count", "keep"}}}},
                {"type": "delta", "mixer": {...}, "mlp": {...}, "weights_of": 0}]}

An optional `max_positions` bounds a request's length (positions are computed, not looked up).
"""
from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, get_float, get_int, get_str

LAYER_TYPES = ("delta", "parallel")
DEFAULT_MAX_POSITIONS = 1 << 16


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: int
    fast: float
    slow: float

    def to_dict(self):
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class SoftmaxSide:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int]
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[RotaryScaling]

    def to_dict(self):
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            rot["scaling"] = self.rot_scaling.to_dict()
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
             "scale": self.scale, "rot": rot}
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        return d


@dataclass(frozen=True)
class LinearSide:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class ParallelMixer:
    left: SoftmaxSide
    right: LinearSide

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class ZuretarMlp:
    kind: str                         # "dense" | "moe"
    ff: int                           # dense: inner width; moe: an expert's inner width
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router = {"experts": self.experts, "top": self.top}
        if self.groups > 1 or self.keep != self.groups:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": router}


@dataclass(frozen=True)
class ZuretarLayer:
    type: str
    mixer: object                     # DeltaMixer | ParallelMixer
    mlp: Optional[ZuretarMlp]
    weights_of: Optional[int] = None

    def to_dict(self):
        d = {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


def _obj(d, key, where):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}.{key} must be an object")
    return v


def _read_delta(m):
    heads, kv = get_int(m, "heads", minimum=1), get_int(m, "kv_heads", minimum=1)
    if heads % kv:
        raise ConfigError(f"config.json: key 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv})")
    return DeltaMixer(heads, kv, get_int(m, "dim", minimum=1), get_int(m, "vdim", minimum=1),
                      get_int(m, "conv", minimum=1))


def _read_left(m, where):
    heads, kv = get_int(m, "heads", minimum=1), get_int(m, "kv_heads", minimum=1)
    if heads % kv:
        raise ConfigError(f"config.json: key 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv})")
    dim = get_int(m, "dim", minimum=1)
    rot = _obj(m, "rot", where)
    dims = get_int(rot, "dims", minimum=0)
    if dims > dim or dims % 2:
        raise ConfigError(f"config.json: key 'dims' ({dims}) must be even and at most 'dim' ({dim})")
    scaling = None
    if rot.get("scaling") is not None:
        sc = _obj(rot, "scaling", where + ".rot")
        scaling = RotaryScaling(get_float(sc, "factor", positive=True), get_int(sc, "original", minimum=1),
                                get_float(sc, "fast", positive=True), get_float(sc, "slow", positive=True))
    chunk = None
    if m.get("mask") is not None:
        chunk = get_int(_obj(m, "mask", where), "size", minimum=1)
    return SoftmaxSide(heads, kv, dim, get_int(m, "vdim", minimum=1), get_float(m, "scale", positive=True), chunk,
                       dims, get_float(rot, "base", positive=True), scaling)


def _read_right(m):
    heads = get_int(m, "heads", minimum=1)
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or not all(
            isinstance(v, (int, float)) and not isinstance(v, bool) for v in decay):
        raise ConfigError(f"config.json: key 'decay' must list one number for each of the {heads} heads")
    return LinearSide(heads, get_int(m, "dim", minimum=1), get_int(m, "vdim", minimum=1), tuple(float(v) for v in decay))


def _read_mlp(mlp, where):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where}.mlp must be null or an object")
    kind = get_str(mlp, "kind", choices={"dense", "moe"})
    if kind == "dense":
        return ZuretarMlp("dense", get_int(mlp, "ff", minimum=1))
    router = _obj(mlp, "router", where + ".mlp")
    experts, top = get_int(router, "experts", minimum=1), get_int(router, "top", minimum=1)
    groups, keep = 1, 1
    if router.get("groups") is not None:
        g = _obj(router, "groups", where + ".mlp.router")
        groups, keep = get_int(g, "count", minimum=1), get_int(g, "keep", minimum=1)
    if experts % groups or keep > groups or top > keep * (experts // groups):
        raise ConfigError(f"config.json: {where}.mlp.router: {experts} experts in {groups} groups, {keep} kept, "
                          f"{top} chosen do not fit together")
    return ZuretarMlp("moe", get_int(_obj(mlp, "expert", where + ".mlp"), "ff", minimum=1), experts, top, groups, keep)


@dataclass(frozen=True)
class ZuretarConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[ZuretarLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[int] = None
    architecture: str = "Zuretar"

    @classmethod
    def from_dict(cls, d):
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: key 'norm' must be an object with 'eps'")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} must be an object with 'type' and 'mixer'")
            kind = get_str(entry, "type", choices=set(LAYER_TYPES))
            m = entry["mixer"]
            try:
                if kind == "delta":
                    mixer = _read_delta(m)
                else:
                    mixer = ParallelMixer(_read_left(_obj(m, "left", where + ".mixer"), where + ".mixer.left"),
                                          _read_right(_obj(m, "right", where + ".mixer")))
                mlp = _read_mlp(entry.get("mlp"), where)
            except ConfigError as e:
                raise ConfigError(f"{e} (in {where})") from None
            src = get_int(entry, "weights_of", default=None, minimum=0)
            layer = ZuretarLayer(kind, mixer, mlp, src)
            if src is not None:
                if src >= i or layers[src].weights_of is not None:
                    raise ConfigError(f"config.json: {where}.weights_of = {src} must name an earlier layer with "
                                      "weights of its own")
                if (layers[src].type, layers[src].mixer, layers[src].mlp) != (kind, mixer, mlp):
                    raise ConfigError(f"config.json: {where} uses the weights of layer {src} but describes "
                                      "another layer")
            layers.append(layer)
        return cls(vocab=get_int(d, "vocab", minimum=1), width=get_int(d, "width", minimum=1),
                   norm_eps=get_float(norm, "eps", positive=True), layers=tuple(layers),
                   max_positions=get_int(d, "max_positions", default=DEFAULT_MAX_POSITIONS, minimum=1),
                   eos_token_id=get_int(d, "eos_token_id", default=None))

    def to_dict(self):
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
