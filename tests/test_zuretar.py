"""Zuretar without a device: configuration, plan, tensors, cache groups with several needs a call,
pages given back behind a chunk, and the plain implementation's own consistency."""
import copy

import numpy as np
import pytest

import plain_zuretar as P
from zuretar_models import ZUR, make_dir


def _cfg(name):
    from sglang_c_b200.config import resolve_architecture
    arch = resolve_architecture(ZUR[name])
    return arch, arch.config_class.from_dict(ZUR[name])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_config_round_trip_and_plan(name):
    from sglang_c_b200.weights.loader import required_tensors
    arch, cfg = _cfg(name)
    assert arch.name == "Zuretar"
    assert arch.config_class.from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict()["layers"] == ZUR[name]["layers"]
    plan = arch.build_plan(cfg)
    need = required_tensors(plan)
    layers = ZUR[name]["layers"]
    E = ZUR[name]["width"]
    assert len(plan.order) == len(layers)
    own = [i for i, layer in enumerate(layers) if "weights_of" not in layer]
    assert len(plan.layers) == len(own)
    for i, layer in enumerate(layers):
        src = layer.get("weights_of", i)
        assert plan.order[i].layer == own.index(src) and plan.order[i].cache_of is None
        if "weights_of" in layer:
            assert not any(k.startswith(f"l{i}.") for k in need)
            continue
        m = layer["mixer"]
        if layer["type"] == "delta":
            assert need[f"l{i}.mix.q"].shape == (m["kv_heads"] * m["dim"], E)
            assert need[f"l{i}.mix.v.conv"].shape == (m["heads"] * m["vdim"], m["conv"])
            assert need[f"l{i}.mix.norm"].shape == (m["vdim"],)
            assert need[f"l{i}.mix.A_log"].shape == (m["heads"],)
        else:
            assert need[f"l{i}.mix.left.v"].shape == (m["left"]["kv_heads"] * m["left"]["vdim"], E)
            assert need[f"l{i}.mix.left.sink"].shape == (m["left"]["heads"],)
            assert need[f"l{i}.mix.right.norm"].shape == (m["right"]["heads"] * m["right"]["vdim"],)
            assert need[f"l{i}.mix.left.out"].shape == need[f"l{i}.mix.right.out"].shape == (E,)
        mlp = layer["mlp"]
        assert (f"l{i}.mlp.gate.b" in need) == (mlp is not None and mlp["kind"] == "dense")
        if mlp is not None and mlp["kind"] == "moe":
            n = mlp["router"]["experts"]
            assert need[f"l{i}.mlp.router"].shape == (n, E) and need[f"l{i}.mlp.correction"].shape == (n,)
            assert need[f"l{i}.mlp.e{n - 1}.down"].shape == (E, mlp["expert"]["ff"]) and f"l{i}.mlp.e{n}.up" not in need
    assert plan.head.weights["weight"] == "head" and plan.embedding.weights["table"] == "embed"


def test_config_errors_name_the_key():
    from sglang_c_b200.config import ConfigError, resolve_architecture
    arch = resolve_architecture(ZUR["A"])

    def broken(change):
        d = copy.deepcopy(ZUR["A"])
        change(d)
        with pytest.raises(ConfigError) as e:
            arch.config_class.from_dict(d)
        return str(e.value)

    assert "type" in broken(lambda d: d["layers"][0].update(type="attention"))
    assert "conv" in broken(lambda d: d["layers"][0]["mixer"].pop("conv"))
    assert "kv_heads" in broken(lambda d: d["layers"][0]["mixer"].update(kv_heads=3))
    assert "decay" in broken(lambda d: d["layers"][1]["mixer"]["right"].update(decay=[0.5]))
    assert "dims" in broken(lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=33))
    assert "weights_of" in broken(lambda d: d["layers"][2].update(weights_of=4))         # not earlier
    assert "weights_of" in broken(lambda d: d["layers"][4].update(weights_of=2))         # no weights of its own
    assert "layer 0" in broken(lambda d: d["layers"][2].update(mixer=dict(d["layers"][2]["mixer"], vdim=8)))   # other sizes
    assert "router" in broken(lambda d: d["layers"][1]["mlp"]["router"].update(top=5))   # more than the kept groups hold
    assert "eps" in broken(lambda d: d["norm"].pop("eps"))


def test_cache_groups_slots_and_chunk_release():
    """A call's need may be a tuple; equal needs share a group; pages of chunks gone by return."""
    from sglang_c_b200.cache import CacheManager
    from sglang_c_b200.cache.needs import CacheNeed
    delta = (CacheNeed.state((2, 4, 3)), CacheNeed.state((3, 10)))
    par = (CacheNeed.paged_kv(2, 8, v_dim=6, chunk=24), CacheNeed.state((1, 5, 7)))
    needs = [delta, par, delta, None, par]
    cm = CacheManager(needs, [None] * 5, page_size=8, n_pages=12, max_requests=3)
    assert len(cm.groups) == 4
    b0, b2, b1, b4 = cm.binding(0), cm.binding(2), cm.binding(1), cm.binding(4)
    assert isinstance(b0, tuple) and len(b0) == 2 and [b.kind for b in b1] == ["paged_kv", "state"]
    assert b0[0].group == b2[0].group and b0[1].group == b2[1].group and b1[0].group == b4[0].group
    assert cm.binding(3) is None
    gi = b1[0].group
    assert cm.add_request("a") is not None and cm.extend("a", 20)
    assert cm.block_table(gi, "a") == [0, 1, 2] and cm.n_free_pages() == 9
    assert cm.extend("a", 30)                      # positions 20..29: the queries at 20..23 still see chunk 0
    assert [p >= 0 for p in cm.block_table(gi, "a")] == [True] * 4
    assert cm.extend("a", 50)                      # from position 30 on nothing before 24 is seen
    assert [p >= 0 for p in cm.block_table(gi, "a")] == [False, False, False, True, True, True, True]
    assert cm.extend("a", 75)                      # ... and from 50 on nothing before 48
    assert [p >= 0 for p in cm.block_table(gi, "a")][:6] == [False] * 6
    cm.check()
    assert cm.add_request("b") is not None and cm.add_request("c") is not None and cm.add_request("d") is None
    cm.free_request("a")
    assert cm.add_request("d") is not None
    cm.check()
    for r in ("b", "c", "d"):
        cm.free_request(r)
    assert cm.n_free_pages() == 12 and cm.n_free_slots() == 3


def test_plain_mechanisms_agree_with_themselves(tmp_path):
    """The oracle's own consistency: a layer that uses another's weights gives that layer's result on the
    same input; the router never chooses outside the kept groups, and its weights are the plain scores;
    a position's logits do not depend on what follows it."""
    d = make_dir(tmp_path, "A")
    cfg, w = P.read_model_dir(d)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((9, cfg["width"]))
    assert np.array_equal(P.layer(x, w, cfg, 0), P.layer(x, w, cfg, 2))
    mlp = cfg["layers"][1]["mlp"]
    h = rng.standard_normal((50, cfg["width"])) * 3
    w2 = dict(w)
    w2["l1.mlp.correction"] = rng.standard_normal(8) - 1.5
    chosen, weight = P.route(h, w2, "l1.mlp.", mlp["router"])
    s = P.sigmoid(h @ w2["l1.mlp.router"].T)
    assert np.allclose(weight, np.take_along_axis(s, chosen, -1))
    for t in range(50):
        groups = {int(e) // 2 for e in chosen[t]}
        assert len(set(chosen[t])) == 2 and len(groups) <= 2
        choice = (s[t] + w2["l1.mlp.correction"]).reshape(4, 2)
        kept = set(np.argsort(-choice.sum(-1), kind="stable")[:2].tolist())
        assert groups <= kept
    toks = [int(t) for t in rng.integers(0, cfg["vocab"], 40)]
    full = P.forward(cfg, w, toks)
    assert np.abs(P.forward(cfg, w, toks[:31]) - full[:31]).max() < 1e-9
