"""Tukavik without a device: configuration, plan, tensors, cache groups, and the plain
implementation's own consistency."""
import copy

import numpy as np
import pytest

import plain_tukavik as P
from tukavik_models import TUK, make_dir


def _cfg(name):
    from sglang_c_b200.config import resolve_architecture
    arch = resolve_architecture(TUK[name])
    return arch, arch.config_class.from_dict(TUK[name])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_config_round_trip_and_plan(name):
    from sglang_c_b200.weights.loader import required_tensors
    arch, cfg = _cfg(name)
    assert arch.name == "Tukavik"
    assert arch.config_class.from_dict(cfg.to_dict()) == cfg
    plan = arch.build_plan(cfg)
    need = required_tensors(plan)
    layers = TUK[name]["layers"]
    assert len(plan.order) == len(layers)
    for i, layer in enumerate(layers):
        assert need[f"l{i}.dwa"].shape == (i + 2,)
        assert (f"l{i}.mlp.up" in need) == (layer["mlp"] is not None)
        assert (f"l{i}.norm2b" in need) == (layer["mlp"] is not None)
        m = layer["mixer"]
        if layer["type"] == "mingru":
            assert need[f"l{i}.mix.z"].shape == (m["width"], TUK[name]["width"])
            assert need[f"l{i}.mix.o"].shape == (TUK[name]["width"], m["width"])
        else:
            assert need[f"l{i}.mix.uk"].shape == (m["heads"] * m["dim"], m["kv_rank"])
            assert need[f"l{i}.mix.uv"].shape == (m["heads"] * m["vdim"], m["kv_rank"])
            assert (f"l{i}.mix.dkv" in need) == ("kv_from" not in m)
            assert (f"l{i}.mix.dq" in need) == (layer["type"] == "latent_attention_2")
            assert plan.order[i].cache_of == m.get("kv_from")
    assert plan.head.weights["weight"] == plan.embedding.weights["table"] == "embed"


def test_config_errors_name_the_key():
    from sglang_c_b200.config import ConfigError, resolve_architecture
    arch = resolve_architecture(TUK["A"])

    def broken(change):
        d = copy.deepcopy(TUK["A"])
        change(d)
        with pytest.raises(ConfigError) as e:
            arch.config_class.from_dict(d)
        return str(e.value)

    assert "type" in broken(lambda d: d["layers"][0].update(type="attention"))
    assert "kv_rank" in broken(lambda d: d["layers"][0]["mixer"].pop("kv_rank"))
    assert "kv_from" in broken(lambda d: d["layers"][3]["mixer"].update(kv_from=1))      # a recurrence
    assert "kv_from" in broken(lambda d: d["layers"][3]["mixer"].update(kv_from=4))      # not earlier
    assert "kv_from" in broken(lambda d: d["layers"][3]["mixer"].update(kv_from=0))      # another rank
    assert "kind" in broken(lambda d: d["layers"][0]["mlp"].update(kind="routed"))
    assert "eps" in broken(lambda d: d["norm"].pop("eps"))
    assert "layers" in broken(lambda d: d.update(layers=[]))


def test_cache_groups_state_slots_and_shared_latents():
    from sglang_c_b200.cache import CacheManager, CacheNeed
    arch, cfg = _cfg("B")
    plan = arch.build_plan(cfg)
    from sglang_c_b200.parts.registry import get_part
    needs = []
    for call in plan.order:
        spec = plan.layers[call.layer].mixer
        needs.append(get_part("mixer", spec.kind)(spec.params, None).cache_need())
    cm = CacheManager(needs, [c.cache_of for c in plan.order], 16, 12, 3)
    kinds = sorted((g.need.kind, g.need.head_dim, len(g.calls)) for g in cm.groups)
    # latents of 64 (one owner; the layer that reads them owns nothing), latents of 128, two recurrences
    # of different widths
    assert kinds == [("paged_kv", 64, 1), ("paged_kv", 128, 1), ("state", 0, 1), ("state", 0, 1)]
    assert all(g.need.shared for g in cm.groups if g.need.kind == "paged_kv")
    assert cm.binding(2).group == cm.binding(1).group and not cm.binding(2).write and cm.binding(1).write
    assert CacheNeed.paged_kv(1, 64, shared=True) != CacheNeed.paged_kv(1, 64)
    # slots and pages come back and are handed out again
    a, b, c = cm.add_request("a"), cm.add_request("b"), cm.add_request("c")
    assert cm.add_request("d") is None
    assert cm.extend("a", 100) and not cm.extend("b", 100)
    cm.free_request("a")
    assert cm.add_request("d") == a and cm.extend("d", 150)
    cm.check()


def test_plain_recurrence_carries_its_state(tmp_path):
    rng = np.random.default_rng(0)
    E, W, n = 12, 20, 37
    h = rng.standard_normal((n, E))
    wz, wx, wg = (rng.standard_normal((W, E)) * 0.3 for _ in range(3))
    bz, bx = rng.standard_normal(W), rng.standard_normal(W)
    wo = rng.standard_normal((E, W)) * 0.3
    whole, s_end = P.min_gru(h, wz, bz, wx, bx, wg, wo)
    first, s_mid = P.min_gru(h[:11], wz, bz, wx, bx, wg, wo)
    rest, s_end2 = P.min_gru(h[11:], wz, bz, wx, bx, wg, wo, state=s_mid)
    assert np.allclose(np.concatenate([first, rest]), whole, atol=1e-12) and np.allclose(s_end, s_end2)
    # the candidate is continuous at 0 and the activation at 0
    assert abs(float(P.xielu(np.array(1e-9), 0.3, -0.2)) - float(P.xielu(np.array(-1e-9), 0.3, -0.2))) < 1e-8
    assert np.allclose(P.sinusoid(3, 7)[2, :2], [np.sin(2.0), np.cos(2.0)])


def test_random_folder_loads_and_runs_plain(tmp_path):
    from sglang_c_b200.config.registry import load_config
    from sglang_c_b200.weights.loader import load_checked
    d = make_dir(tmp_path, "C")
    arch, cfg = load_config(d)
    refs = load_checked(arch.build_plan(cfg), d)
    assert "l0.mix.dq.norm" in refs and "final.norm" in refs
    logits = P.forward_dir(d, [3, 1, 4, 1, 5, 9, 2, 6])
    assert logits.shape == (8, TUK["C"]["vocab"]) and np.isfinite(logits).all()
    # causal: the logits of a prefix do not depend on what follows
    assert np.allclose(P.forward_dir(d, [3, 1, 4, 1, 5])[:5], logits[:5], atol=1e-10)
