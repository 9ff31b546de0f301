"""Typed configuration of the Tukavik architecture: a decoder whose config.json lists its
layers one by one, each with the kind of its mixer (a minGRU recurrence, or attention over a
cached latent with direct or low-rank queries), the mixer's sizes, and an optional dense
feed-forward.  Every size and every constant that may differ between models comes from the file:

    {"architecture": "Tukavik", "vocab": V, "width": E, "norm": {"eps": e},
     "layers": [{"type": "mingru", "mixer": {"width": W}, "mlp": null},
                {"type": "latent_attention", "mixer": {"heads", "dim", "vdim", "kv_rank", "scale"},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "latent_attention_2", "mixer": {... , "q_rank", optional "kv_from": j}, "mlp": ...}]}

`kv_from: j` makes an attention layer (of either kind) read the latents layer j caches instead of
projecting its own.
An optional `max_positions` bounds a request's length (positions are computed, not looked up,
so the architecture itself has no bound).
"""
from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, get_float, get_int, get_str

LAYER_TYPES = ("mingru", "latent_attention", "latent_attention_2")
DEFAULT_MAX_POSITIONS = 1 << 16


@dataclass(frozen=True)
class TukavikLayer:
    type: str
    width: int = 0                    # mingru: channels of the recurrence
    heads: int = 0                    # latent attention ...
    dim: int = 0                      # query/key size per head
    vdim: int = 0                     # value size per head
    kv_rank: int = 0                  # the cached latent's size
    q_rank: Optional[int] = None      # latent_attention_2: the queries' latent
    scale: float = 0.0                # multiplier of q·k
    kv_from: Optional[int] = None     # read this layer's latents
    ff: Optional[int] = None          # feed-forward width; None: the layer has no feed-forward

    def to_dict(self):
        if self.type == "mingru":
            mixer = {"width": self.width}
        else:
            mixer = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                     "scale": self.scale}
            if self.type == "latent_attention_2":
                mixer["q_rank"] = self.q_rank
            if self.kv_from is not None:
                mixer["kv_from"] = self.kv_from
        mlp = None if self.ff is None else {"kind": "dense", "ff": self.ff}
        return {"type": self.type, "mixer": mixer, "mlp": mlp}


@dataclass(frozen=True)
class TukavikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[TukavikLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[int] = None
    architecture: str = "Tukavik"

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
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}.mlp must be null or an object")
                get_str(mlp, "kind", choices={"dense"})
                ff = get_int(mlp, "ff", minimum=1)
            try:
                if kind == "mingru":
                    layers.append(TukavikLayer(kind, width=get_int(m, "width", minimum=1), ff=ff))
                    continue
                kv_from = get_int(m, "kv_from", default=None, minimum=0)
                dim = get_int(m, "dim", minimum=1)
                layer = TukavikLayer(
                    kind, heads=get_int(m, "heads", minimum=1), dim=dim,
                    vdim=get_int(m, "vdim", minimum=1), kv_rank=get_int(m, "kv_rank", minimum=1),
                    q_rank=get_int(m, "q_rank", minimum=1) if kind == "latent_attention_2" else None,
                    # (a file that leaves the multiplier out means the usual 1/sqrt(dim))
                    scale=get_float(m, "scale", default=dim ** -0.5, positive=True), kv_from=kv_from, ff=ff)
            except ConfigError as e:
                raise ConfigError(f"{e} (in {where}.mixer)") from None
            if kv_from is not None:
                src = layers[kv_from] if kv_from < i else None
                if src is None or src.type == "mingru" or src.kv_from is not None or src.kv_rank != layer.kv_rank:
                    raise ConfigError(f"config.json: {where}.mixer.kv_from = {kv_from} must name an earlier layer "
                                      "that projects a latent of the same kv_rank itself")
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
