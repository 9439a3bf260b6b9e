"""The Vokepel configuration reader and the description it builds (no device needed)."""
import copy

import pytest

from vokepel_helpers import CONFIG_A, CONFIG_B, CONFIG_C, config, dense, left_side, pair, talking
from purhie_b200.config import ConfigError, ModelConfig, registered_architectures, registered_parts
from purhie_b200.weights import expected_tensors


def test_the_architecture_and_its_parts_are_registered():
    assert "Vokepel" in registered_architectures()
    assert {"talking_attention", "min_gru", "side_by_side", "attention"} <= set(registered_parts("mixer"))
    assert "mlp" in registered_parts("feed_forward") and "rmsnorm" in registered_parts("norm")


def test_the_description_follows_the_layer_list():
    cfg = ModelConfig.from_dict(CONFIG_A)
    assert cfg.architecture == "Vokepel"
    spec = cfg.model_spec()
    layers = spec["layers"]
    kinds = [(l["arrangement"], l["parts"].get("mixer", {}).get("kind"), l["parts"].get("feed_forward", {}).get("kind")) for l in layers]
    assert kinds == [("pre_norm", "side_by_side", "mlp"), ("pre_norm", "talking_attention", None), ("pre_norm", "talking_attention", "mlp"),
                     ("pre_norm", "side_by_side", "mlp"), ("reinject", None, None)]
    for l in layers[:4]:
        assert l["params"]["residual_factor"] == 0.6
        assert l["parts"]["mixer_norm"]["kind"] == "rmsnorm" and l["parts"]["mixer_norm"]["params"]["eps"] == 1e-6
    assert "feed_forward_norm" not in layers[1]["parts"]
    t = layers[1]["parts"]["mixer"]["params"]
    assert (t["num_heads"], t["num_kv_heads"], t["head_dim"], t["value_dim"], t["window"], t["scale"], t["softcap"]) == (4, 2, 12, 12, 21, 0.3, 5.0)
    assert t["values"] == "keys" and t["joint_norm_eps"] == 1e-6
    assert set(t["names"]) == {"q_proj", "k_proj", "o_proj", "q_norm", "k_norm", "distance_slope", "distance_rate", "head_mix", "gate_proj"}
    assert layers[2]["parts"]["mixer"]["params"]["softcap"] is None
    s = layers[0]["parts"]["mixer"]["params"]
    assert (s["combine"], s["left_factor"], s["right_factor"]) == ("weighted_sum", 0.8, 1.3)
    a = s["left"]["params"]
    assert s["left"]["kind"] == "attention" and (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["value_dim"], a["window"]) == (3, 1, 8, 12, 13)
    assert a["position"]["params"] == {"theta": 500.0, "n_rot": 4, "max_position": 65536, "pairing": "interleaved"}
    assert a["qk_norm_eps"] is None and a["names"]["sink"] == "l0.mix.left.sink"
    assert s["right"]["kind"] == "min_gru" and s["right"]["params"]["width"] == 40
    assert layers[3]["parts"]["mixer"]["params"]["left"]["params"]["window"] == 0
    assert layers[0]["parts"]["feed_forward"]["params"]["activation"] == "relu2"
    h = spec["head"]["params"]
    assert (h["tied_to"], h["scale"], h["softcap"]) == ("embed", 1.7, 12.0) and spec["keep_embedding_output"] is True
    plain = ModelConfig.from_dict(CONFIG_B).model_spec()
    assert plain["head"]["params"]["scale"] == 1.0 and plain["head"]["params"]["softcap"] is None
    assert plain["layers"][0]["params"]["residual_factor"] == 1.0
    assert ModelConfig.from_dict(CONFIG_C).model_spec()["layers"][2]["parts"]["mixer"]["params"]["left"]["params"]["position"] is None


def test_the_run_order_repeats_the_stretch_with_a_reinjection_in_front_of_every_round():
    def order(cfg):
        return [(c["layer"], c["pass"]) for c in ModelConfig.from_dict(cfg).model_spec()["schedule"]]
    assert order(CONFIG_A) == [(0, 0), (4, 0), (1, 0), (2, 0), (4, 1), (1, 1), (2, 1), (3, 0)]          # layer 4: the reinjection
    assert order(CONFIG_B) == [(3, 0), (0, 0), (3, 1), (0, 1), (3, 2), (0, 2), (1, 0), (2, 0)]
    assert order(CONFIG_C) == [(3, 0), (0, 0), (1, 0), (2, 0)]
    straight = copy.deepcopy(CONFIG_B)
    del straight["loop"]
    spec = ModelConfig.from_dict(straight).model_spec()
    assert [(c["layer"], c["pass"]) for c in spec["schedule"]] == [(0, 0), (1, 0), (2, 0)]
    assert len(spec["layers"]) == 3 and spec["keep_embedding_output"] is False
    assert "loop.in" not in expected_tensors(straight)
    assert all(c["cache_from"] is None for c in ModelConfig.from_dict(CONFIG_A).model_spec()["schedule"])


def test_the_tensor_list_has_every_name_with_its_shape():
    t = expected_tensors(CONFIG_A)
    shape = lambda n: tuple(t[n].shape)
    assert shape("embed") == (80, 48) and shape("final.norm") == (48,) and "head" not in t
    assert shape("loop.in") == (48, 96) and shape("loop.step") == (2, 48)
    assert shape("l1.mix.q") == (48, 48) and shape("l1.mix.k") == (24, 48) and shape("l1.mix.q.norm") == (48,) and shape("l1.mix.k.norm") == (24,)
    assert shape("l1.mix.r1") == (4,) and shape("l1.mix.r2") == (4,) and shape("l1.mix.talk") == (4, 4)
    assert shape("l1.mix.g") == (48, 48) and shape("l1.mix.o") == (48, 48) and "l1.mix.v" not in t
    assert "l1.norm2" not in t and "l1.mlp.up" not in t
    assert shape("l0.mix.left.q") == (24, 48) and shape("l0.mix.left.k") == (8, 48) and shape("l0.mix.left.v") == (12, 48)
    assert shape("l0.mix.left.sink") == (3,) and shape("l0.mix.left.o") == (48, 36)
    assert shape("l0.mix.right.z") == (40, 48) and shape("l0.mix.right.z.b") == (40,) and shape("l0.mix.right.x.b") == (40,)
    assert shape("l0.mix.right.g") == (40, 48) and shape("l0.mix.right.o") == (48, 40)
    assert shape("l0.mlp.up") == (64, 48) and shape("l0.mlp.down") == (48, 64) and shape("l0.norm2") == (48,)
    assert not [n for n in t if "gate" in n or n.endswith(".b") and ".right." not in n]


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="lightning"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=16), "vdim"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(softcap=0.0), "softcap"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=10), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=3), "dims"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["loop"].update(stop=5), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_a_configuration_that_does_not_fit_is_refused_by_name(change, word):
    c = copy.deepcopy(CONFIG_A)
    change(c)
    with pytest.raises(ConfigError) as e:
        ModelConfig.from_dict(c)
    assert word in str(e.value)


def test_a_random_model_folder_of_this_design_is_written_and_passes_the_folder_check(tmp_path):
    from purhie_b200.config import load_config
    from purhie_b200.weights import check_model_folder, list_tensors, write_random_model
    write_random_model(str(tmp_path), CONFIG_B, seed=3, std=0.05, scale_low=0.8, scale_high=1.2, dtype="bfloat16")
    check_model_folder(str(tmp_path))
    names = {t["name"]: t for t in list_tensors(str(tmp_path))}
    assert set(names) == set(expected_tensors(CONFIG_B))
    assert names["loop.step"]["shape"] == [3, 40] and names["l0.mix.talk"]["shape"] == [5, 5] and names["l1.mix.right.z"]["shape"] == [24, 40]
    assert load_config(str(tmp_path)).to_dict()["layers"] == CONFIG_B["layers"]


def test_what_each_mixer_asks_the_cache_manager_for():
    from purhie_b200.parts import PartProbe
    cfg = config(32, 20, [(talking(4, 2, 8, 11), None), (pair(left_side(2, 1, 8, 12, 5, 4), 20), dense(16))])
    spec = ModelConfig.from_dict(cfg).model_spec()
    need = [PartProbe("mixer", l["parts"]["mixer"]["kind"], l["parts"]["mixer"]["params"]).cache_need() for l in spec["layers"]]
    # the talking mixer keeps its normed keys and, as values, the keys as projected: pages of two rows of 8 per kv head
    assert (need[0]["kind"], need[0]["kv_heads"], need[0]["head_dim"], need[0]["window"]) == ("pages", 2, 8, 11) and not need[0]["state_shape"]
    # the pair keeps the left side's pages (values of 12) and the right side's state, one number per channel
    assert (need[1]["kind"], need[1]["kv_heads"], need[1]["head_dim"], need[1]["value_dim"], need[1]["window"]) == ("pages", 1, 8, 12, 5)
    assert need[1]["state_shape"] == [20]
