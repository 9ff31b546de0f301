"""Zuretar as a plan of parts: a token table; layers with one RMS norm that a mixer and a
feed-forward both read, x += mixer(norm(x)) + ff(norm(x)); the mixer is a gated delta rule, or
softmax attention (rotary positions with YaRN scaling, unit-RMS queries and keys, a chunk mask,
a sink per head) side by side with a linear attention of fixed decay; the feed-forward is a gated
MLP with biases, a routed mixture of experts, or absent; a final RMS norm and a head of its own.
A layer that names another's weights is a second call of that layer in the running order, with a
cache and state of its own.

Tensor names: `embed`, `final.norm`, `head`, and for layer i `l<i>.norm1`, `l<i>.mix.*` (delta: q,
q.conv, k, k.conv, v, v.conv, b, a, A_log, dt_bias, g, norm, o; parallel: left.q|k|v|o|sink|out,
right.q|k|v|g|norm|o|out) and `l<i>.mlp.*` (dense: gate, gate.b, up, up.b, down, down.b; experts:
router, correction, e<j>.gate|up|down).
"""
from ..config.registry import register_architecture
from ..config.zuretar import ZuretarConfig
from ..parts.plan import LayerCall, LayerPlan, ModelPlan, PartSpec


def _delta(cfg, m, p):
    return PartSpec("gated_delta",
                    {"size": cfg.width, "n_heads": m.heads, "n_qk_heads": m.kv_heads, "dim": m.dim, "v_dim": m.vdim,
                     "conv": m.conv, "eps": cfg.norm_eps},
                    {"q_weight": p + "q", "q_conv": p + "q.conv", "k_weight": p + "k", "k_conv": p + "k.conv",
                     "v_weight": p + "v", "v_conv": p + "v.conv", "beta_weight": p + "b", "a_weight": p + "a",
                     "A_log": p + "A_log", "dt_bias": p + "dt_bias", "gate_weight": p + "g", "norm": p + "norm",
                     "out_weight": p + "o"})


def _parallel(cfg, m, p):
    le, ri = m.left, m.right
    rot = {"dims": le.rot_dims, "base": le.rot_base,
           "scaling": None if le.rot_scaling is None else le.rot_scaling.to_dict()}
    left = ("rotary_attention", {"size": cfg.width, "n_heads": le.heads, "n_kv_heads": le.kv_heads, "head_dim": le.dim,
                                 "v_dim": le.vdim, "scale": le.scale, "rotary": rot, "qk_norm": True,
                                 "eps": cfg.norm_eps, "chunk": le.chunk, "window": None, "sink": True})
    right = ("linear_decay_attention", {"size": cfg.width, "n_heads": ri.heads, "dim": ri.dim, "v_dim": ri.vdim,
                                        "decay": list(ri.decay), "eps": cfg.norm_eps})
    w = {"left.q_weight": p + "left.q", "left.k_weight": p + "left.k", "left.v_weight": p + "left.v",
         "left.out_weight": p + "left.o", "left.sink": p + "left.sink", "left_out": p + "left.out",
         "right.q_weight": p + "right.q", "right.k_weight": p + "right.k", "right.v_weight": p + "right.v",
         "right.gate_weight": p + "right.g", "right.norm": p + "right.norm", "right.out_weight": p + "right.o",
         "right_out": p + "right.out"}
    return PartSpec("side_by_side", {"size": cfg.width, "eps": cfg.norm_eps, "left": left, "right": right}, w)


def _mlp(cfg, mlp, p):
    if mlp is None:
        return None
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", {"size": cfg.width, "inner_size": mlp.ff, "bias": True},
                        {"gate_weight": p + "gate", "gate_bias": p + "gate.b", "up_weight": p + "up",
                         "up_bias": p + "up.b", "down_weight": p + "down", "down_bias": p + "down.b"})
    w = {"router": p + "router", "correction": p + "correction"}
    for e in range(mlp.experts):
        w.update({f"gate_{e}": f"{p}e{e}.gate", f"up_{e}": f"{p}e{e}.up", f"down_{e}": f"{p}e{e}.down"})
    return PartSpec("routed_experts", {"size": cfg.width, "inner_size": mlp.ff, "n_experts": mlp.experts, "top": mlp.top,
                                       "n_groups": mlp.groups, "keep": mlp.keep}, w)


def build_plan(cfg: ZuretarConfig) -> ModelPlan:
    E = cfg.width
    norm = lambda name: PartSpec("rms_norm", {"size": E, "eps": cfg.norm_eps}, {"weight": name})
    layers, order, built = [], [], {}
    for i, lc in enumerate(cfg.layers):
        if lc.weights_of is not None:
            order.append(LayerCall(built[lc.weights_of]))
            continue
        p = f"l{i}."
        mixer = _delta(cfg, lc.mixer, p + "mix.") if lc.type == "delta" else _parallel(cfg, lc.mixer, p + "mix.")
        built[i] = len(layers)
        layers.append(LayerPlan(name=f"l{i}", block=PartSpec("parallel_sublayers"), norm1=norm(p + "norm1"), mixer=mixer,
                                ffn=_mlp(cfg, lc.mlp, p + "mlp.")))
        order.append(LayerCall(built[i]))
    return ModelPlan(
        hidden_size=E, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "size": E}, {"table": "embed"}),
        position=PartSpec("none", {}, {}),
        layers=layers, order=order, final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "size": E}, {"weight": "head"}),
        eos_token_id=cfg.eos_token_id)


register_architecture("Zuretar", ZuretarConfig, build_plan, model_types=("zuretar",))
