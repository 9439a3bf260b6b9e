"""The Zerusun configuration reader and the description it builds (no device needed)."""
import copy

import pytest

from zerusun_helpers import CONFIG_A, CONFIG_B, config, dense, latent, lightning
from purhie_b200.config import ConfigError, ModelConfig, registered_architectures, registered_parts
from purhie_b200.weights import expected_tensors


def test_the_architecture_and_its_parts_are_registered():
    assert "Zerusun" in registered_architectures()
    assert "dyntanh" in registered_parts("norm")
    assert {"lightning_attention", "latent_attention"} <= set(registered_parts("mixer"))
    assert {"swiglu", "routed_glu"} <= set(registered_parts("feed_forward"))


def test_the_description_follows_the_layer_list():
    cfg = ModelConfig.from_dict(CONFIG_A)
    assert cfg.architecture == "Zerusun"
    spec = cfg.model_spec()
    layers = spec["layers"]
    kinds = [(l["arrangement"], l["parts"].get("mixer", {}).get("kind"), l["parts"].get("feed_forward", {}).get("kind")) for l in layers]
    assert kinds == [("parallel", "latent_attention", "routed_glu"), ("parallel", "lightning_attention", "swiglu"),
                     ("parallel", "lightning_attention", None), ("parallel", "latent_attention", "routed_glu"), ("reinject", None, None)]
    for l in layers[:4]:
        assert l["parts"]["norm"]["kind"] == "dyntanh" and set(l["parts"]["norm"]["params"]["names"]) == {"weight", "bias", "alpha"}
    a = layers[0]["parts"]["mixer"]["params"]
    assert (a["num_heads"], a["head_dim"], a["rot_dim"], a["value_dim"], a["q_rank"], a["kv_rank"]) == (3, 8, 4, 12, 10, 20)
    assert a["window"] == 13 and a["scale"] == 0.4 and a["gate"] is True and a["norm_eps"] == 1e-6
    assert a["position"]["params"] == {"theta": 500.0, "n_rot": 4, "max_position": 65536, "pairing": "half",
                                       "scaling": {"kind": "yarn", "factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}}
    assert "scaling" not in layers[3]["parts"]["mixer"]["params"]["position"]["params"]
    r = layers[2]["parts"]["mixer"]["params"]
    assert (r["num_heads"], r["head_dim"], r["value_dim"], r["decay"]) == (3, 24, 8, [1.0, 0.8, 0.93])
    f = layers[0]["parts"]["feed_forward"]["params"]
    assert (f["experts"], f["top"]) == (6, 2) and f["scoring"] == {"kind": "softmax", "groups": 3, "keep": 2, "scale": 1.5}
    assert f["shared"]["kind"] == "swiglu" and f["shared"]["params"]["intermediate_size"] == 24 and f["names"]["shared_gate"] == "l0.mlp.shared.sg"
    assert "shared" not in layers[3]["parts"]["feed_forward"]["params"] and "shared_gate" not in layers[3]["parts"]["feed_forward"]["params"]["names"]
    assert layers[1]["parts"]["feed_forward"]["params"]["activation"] == {"kind": "gelu_tanh"}
    assert spec["final_norm"]["kind"] == "dyntanh" and spec["embedding"]["params"]["norm"]["kind"] == "dyntanh"
    assert spec["head"]["params"]["tied_to"] == "embed" and spec["keep_embedding_output"] is True


def test_the_run_order_repeats_the_stretch_with_a_reinjection_in_front_of_every_round():
    def order(cfg):
        return [(c["layer"], c["pass"]) for c in ModelConfig.from_dict(cfg).model_spec()["schedule"]]
    assert order(CONFIG_A) == [(0, 0), (4, 0), (1, 0), (2, 0), (4, 1), (1, 1), (2, 1), (3, 0)]          # layer 4: the reinjection
    assert order(CONFIG_B) == [(3, 0), (0, 0), (3, 1), (0, 1), (3, 2), (0, 2), (1, 0), (2, 0)]
    whole = copy.deepcopy(CONFIG_B)
    whole["loop"] = {"start": 0, "stop": 3, "times": 1}
    assert order(whole) == [(3, 0), (0, 0), (1, 0), (2, 0)]
    straight = copy.deepcopy(CONFIG_B)
    del straight["loop"]
    spec = ModelConfig.from_dict(straight).model_spec()
    assert [(c["layer"], c["pass"]) for c in spec["schedule"]] == [(0, 0), (1, 0), (2, 0)]
    assert len(spec["layers"]) == 3 and spec["keep_embedding_output"] is False
    assert "loop.in" not in expected_tensors(straight)
    # every entry of the run order keeps a cache of its own
    assert all(c["cache_from"] is None for c in ModelConfig.from_dict(CONFIG_A).model_spec()["schedule"])


def test_the_tensor_list_has_every_name_with_its_shape():
    t = expected_tensors(CONFIG_A)
    shape = lambda n: tuple(t[n].shape)
    assert shape("embed") == (80, 48) and "head" not in t and shape("final.norm") == (48,) and shape("final.norm.b") == (48,)
    assert shape("embed.norm.alpha") == () and shape("l2.norm1.alpha") == ()
    assert shape("loop.in") == (48, 96) and shape("loop.step") == (2, 48)
    assert shape("l0.mix.dq") == (10, 48) and shape("l0.mix.dq.norm") == (10,) and shape("l0.mix.uq") == (36, 10)
    assert shape("l0.mix.dkv") == (24, 48) and shape("l0.mix.dkv.norm") == (20,)
    assert shape("l0.mix.uk") == (24, 20) and shape("l0.mix.uv") == (36, 20) and shape("l0.mix.g") == (3, 48) and shape("l0.mix.o") == (48, 36)
    assert shape("l1.mix.q") == (16, 48) and shape("l1.mix.v") == (32, 48) and shape("l1.mix.g") == (32, 48)
    assert shape("l1.mix.norm") == (32,) and shape("l1.mix.o") == (48, 32)
    assert shape("l0.mlp.router") == (6, 48) and shape("l0.mlp.e5.gate") == (16, 48) and shape("l0.mlp.e5.down") == (48, 16)
    assert shape("l0.mlp.shared.up") == (24, 48) and shape("l0.mlp.shared.sg") == (1, 48)
    assert "l3.mlp.shared.sg" not in t and "l3.mlp.shared.up" not in t
    assert shape("l1.mlp.gate") == (64, 48) and "l2.mlp.up" not in t and "l2.norm2" not in t


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 1.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "dims"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.0), "factor"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["loop"].update(stop=5), "loop"),
    (lambda c: c["loop"].update(start=3), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.pop("width"), "width"),
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
    assert names["loop.step"]["shape"] == [3, 40] and names["l1.norm1.alpha"]["shape"] == [] and names["l2.mix.uq"]["shape"] == [30, 16]
    assert load_config(str(tmp_path)).to_dict()["layers"] == CONFIG_B["layers"]


def test_a_latent_mixer_asks_for_rows_without_values_and_a_lightning_mixer_for_a_state():
    cfg = config(32, 20, [(latent(2, 8, 4, 8, 8, 12, 5), None), (lightning(3, 20, 6, [0.9, 0.9, 0.9]), dense(16))])
    spec = ModelConfig.from_dict(cfg).model_spec()
    assert [l["parts"]["mixer"]["kind"] for l in spec["layers"]] == ["latent_attention", "lightning_attention"]
    assert "feed_forward" not in spec["layers"][0]["parts"]
