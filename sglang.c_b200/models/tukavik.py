"""Tukavik as a plan of parts: a token table plus a sinusoidal position vector; layers with a
norm ahead of and behind each sublayer, whose mixer is a minGRU recurrence or attention over a
cached latent (queries direct or through a latent of their own; a layer may read another layer's
latents), with or without a dense feed-forward under an xIELU activation; behind every layer a
weighted average of all layers' results so far; a final norm and a head tied to the token table.

Tensor names: `embed`, `final.norm`, and for layer i `l<i>.norm1|norm1b|norm2|norm2b`,
`l<i>.dwa`, `l<i>.mix.*` (minGRU: z, z.b, x, x.b, g, o; attention: q | dq, dq.norm, uq; dkv,
dkv.norm, uk, uv, o) and `l<i>.mlp.up|down|act`.
"""
from ..config.registry import register_architecture
from ..config.tukavik import TukavikConfig
from ..parts.plan import LayerCall, LayerPlan, ModelPlan, PartSpec

SINUSOID_BASE = 10000.0


def build_plan(cfg: TukavikConfig) -> ModelPlan:
    E, L = cfg.width, len(cfg.layers)
    norm = lambda name: PartSpec("layer_norm", {"size": E, "eps": cfg.norm_eps, "bias": False}, {"weight": name})
    layers, order = [], []
    for i, lc in enumerate(cfg.layers):
        p = f"l{i}."
        if lc.type == "mingru":
            mixer = PartSpec("min_gru", {"size": E, "width": lc.width},
                             {"gate_weight": p + "mix.z", "gate_bias": p + "mix.z.b", "cand_weight": p + "mix.x",
                              "cand_bias": p + "mix.x.b", "out_gate_weight": p + "mix.g", "out_weight": p + "mix.o"})
        else:
            own = lc.kv_from is None
            w = {"k_up": p + "mix.uk", "v_up": p + "mix.uv", "out_weight": p + "mix.o"}
            if lc.q_rank:
                w.update({"q_down": p + "mix.dq", "q_norm": p + "mix.dq.norm", "q_up": p + "mix.uq"})
            else:
                w["q_weight"] = p + "mix.q"
            if own:
                w.update({"kv_down": p + "mix.dkv", "kv_norm": p + "mix.dkv.norm"})
            mixer = PartSpec("latent_attention",
                             {"size": E, "n_heads": lc.heads, "qk_dim": lc.dim, "v_dim": lc.vdim,
                              "kv_rank": lc.kv_rank, "q_rank": lc.q_rank, "scale": lc.scale, "eps": cfg.norm_eps,
                              "own_latent": own, "window": None}, w)
        parts = {"norm1b": ("norm", norm(p + "norm1b")),
                 "depth_mix": ("stream_mix", PartSpec("depth_weighted_average", {"index": i, "n_layers": L, "size": E},
                                                      {"weights": p + "dwa"}))}
        ffn = None
        if lc.ff is not None:
            ffn = PartSpec("mlp", {"size": E, "inner_size": lc.ff, "activation": "xielu", "bias": False,
                                   "weight_layout": "linear"},
                           {"up_weight": p + "mlp.up", "down_weight": p + "mlp.down", "act_params": p + "mlp.act"})
            parts["norm2b"] = ("norm", norm(p + "norm2b"))
        layers.append(LayerPlan(name=f"l{i}", block=PartSpec("sandwich_norm"), norm1=norm(p + "norm1"), mixer=mixer,
                                norm2=norm(p + "norm2") if ffn is not None else None, ffn=ffn, parts=parts))
        order.append(LayerCall(i, cache_of=lc.kv_from))
    return ModelPlan(
        hidden_size=E, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "size": E}, {"table": "embed"}),
        position=PartSpec("sinusoidal", {"size": E, "base": SINUSOID_BASE}, {}),
        layers=layers, order=order, final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "size": E}, {"weight": "embed"}),
        eos_token_id=cfg.eos_token_id)


register_architecture("Tukavik", TukavikConfig, build_plan, model_types=("tukavik",))
