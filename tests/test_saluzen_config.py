"""The Saluzen configuration on the host, without a GPU: reading config.json, what it refuses, the model spec it becomes
(pairs of mixers, shared latents as a schedule), and the check of a checkpoint against it."""
import copy

import pytest

from saluzen_cases import CASES, CASE_A, CASE_B, CASE_C, random_weights, tensor_shapes, write_model


def test_registered_and_chosen_by_name():
    from fastgguf_b200.config import SaluzenConfig
    from fastgguf_b200.registry import config_from_dict, registered_architectures
    assert "Saluzen" in registered_architectures()
    cfg = config_from_dict(CASE_A)
    assert isinstance(cfg, SaluzenConfig) and cfg.architecture == "Saluzen"
    assert cfg.to_dict() == CASE_A
    d = cfg.describe()
    assert d["hidden_size"] == 96 and d["vocab_size"] == 211 and d["num_hidden_layers"] == 4 and d["layer_runs"] == 4
    assert d["layer_kinds"] == ["latent_attention+dense", "parallel+dense", "latent_attention+none", "parallel_2+dense"]
    # the first latent layer's latent and rotated part (the third reads them), and the two left sides' keys and values
    assert d["kv_bytes_per_token"]["bfloat16"] == 2 * ((40 + 8) + 2 * (24 + 40) + 3 * (16 + 16))
    ssm_state = 3 * (3 * 24 + 2 * 16) + 3 * 16 * 24
    delta_state = 1 * (2 * 2 * 16 + 4 * 24) + 4 * 16 * 24
    assert d["state_bytes_per_sequence"] == 4 * (ssm_state + delta_state)
    # every tensor of the folder is counted
    import math
    assert d["parameters"] == sum(math.prod(s) for s in tensor_shapes(CASE_A).values())


def test_shared_latents_become_a_schedule():
    from fastgguf_b200.registry import config_from_dict
    spec = config_from_dict(CASE_A).spec_json()
    assert [(r["layer"], r["cache_from"]) for r in spec["schedule"]] == [(0, None), (1, None), (2, 0), (3, None)]
    assert spec["layers"][2]["mixer"]["params"]["shared_kv"] is True and "kv_down.weight" not in spec["layers"][2]["mixer"]["tensors"]
    assert spec["layers"][0]["mixer"]["params"]["shared_kv"] is False and spec["layers"][0]["mixer"]["tensors"]["kv_down.weight"] == "l0.mix.dkv"
    b = config_from_dict(CASE_B).spec_json()
    assert [r["cache_from"] for r in b["schedule"]] == [None, None, None, None, 2]


def test_spec_follows_the_file():
    from fastgguf_b200.registry import config_from_dict
    spec = config_from_dict(CASE_A).spec_json()
    kinds = [(l["block"], l["mixer"]["kind"], (l["feed_forward"] or {}).get("kind")) for l in spec["layers"]]
    assert kinds == [("sandwich", "latent_attention", "swiglu"), ("sandwich", "mixer_pair", "swiglu"), ("sandwich", "latent_attention", None),
                     ("sandwich", "mixer_pair", "swiglu")]
    assert all(l["mixer_post_norm"]["tensors"]["weight"] == f"l{i}.norm1b" for i, l in enumerate(spec["layers"]))
    assert spec["layers"][1]["feed_forward_post_norm"]["tensors"]["weight"] == "l1.norm2b" and spec["layers"][2].get("feed_forward_post_norm") is None
    p = spec["layers"][1]["mixer"]["params"]
    assert p["normalize"] is True and p["left_scale"] == 0.5 and p["right_scale"] == 0.5 and p["eps"] == 1e-6
    a = p["left"]["params"]
    assert p["left"]["kind"] == "sink_attention" and (a["n_heads"], a["n_kv_heads"], a["head_dim"], a["v_head_dim"], a["scale"], a["chunk"]) == (4, 2, 24, 40, 0.3, 0)
    assert a["unit_sink"] is True and "sink" not in a and a["gate"] == "full" and a["bias"] is True
    assert a["position"]["params"] == {"head_dim": 24, "theta": 10000.0, "rotary_dim": 8, "layout": "halves", "scaling": None}
    r = p["right"]["params"]
    assert p["right"]["kind"] == "state_space" and (r["n_heads"], r["v_head_dim"], r["state_size"], r["n_groups"], r["conv_taps"], r["norm_groups"]) == (3, 24, 16, 1, 4, 1)
    t = spec["layers"][1]["mixer"]["tensors"]
    assert t["left.q_proj.bias"] == "l1.mix.left.q.b" and t["right.in_proj.weight"] == "l1.mix.right.in" and t["left_norm.weight"] == "l1.mix.left.out"
    assert t["right.conv.bias"] == "l1.mix.right.conv.b" and "left.sinks" not in t
    p = spec["layers"][3]["mixer"]["params"]
    assert p["normalize"] is False and p["left_scale"] == 0.7 and p["right_scale"] == 1.3
    a = p["left"]["params"]
    assert a["sink"] is True and "unit_sink" not in a and a["gate"] == "head" and a["chunk"] == 9
    r = p["right"]["params"]
    assert p["right"]["kind"] == "gated_delta" and (r["n_heads"], r["n_kv_heads"], r["head_dim"], r["v_head_dim"], r["conv_taps"]) == (4, 2, 16, 24, 2)
    assert r["unit_eps"] == 1e-6 and r["q_scale"] == 0.25
    t = spec["layers"][3]["mixer"]["tensors"]
    assert t["left.sinks"] == "l3.mix.left.sink" and t["right.b_proj.weight"] == "l3.mix.right.b" and t["right.q_conv.weight"] == "l3.mix.right.q.conv"
    m = spec["layers"][0]["mixer"]["params"]
    assert (m["rot_dim"], m["kv_rank"], m["q_rank"], m["head_dim"], m["v_head_dim"]) == (8, 40, 48, 16, 24) and not m["sink"] and not m["gate"]
    assert m["position"]["params"]["layout"] == "adjacent"
    scaled = config_from_dict(CASE_B).spec_json()["layers"][1]["mixer"]["params"]["left"]["params"]["position"]["params"]["scaling"]
    assert scaled == {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64.0}
    assert config_from_dict(CASE_B).spec_json()["layers"][3]["mixer"]["params"]["left"]["params"]["position"] is None
    assert spec["head"]["tensors"]["weight"] == "head" and spec["embedding"]["tensors"]["weight"] == "embed"


def test_python_spec_round_trip():
    from fastgguf_b200.engine.spec import ModelSpec
    from fastgguf_b200.registry import config_from_dict
    j = config_from_dict(CASE_A).spec_json()
    again = ModelSpec.from_json(j).to_json()
    assert again["schedule"] == j["schedule"]
    pair, back = j["layers"][1]["mixer"], again["layers"][1]["mixer"]
    assert back["kind"] == "mixer_pair" and back["tensors"] == pair["tensors"]
    for side in ("left", "right"):
        assert back["params"][side]["kind"] == pair["params"][side]["kind"] and back["params"][side]["params"] == pair["params"][side]["params"]
    assert again["layers"][2]["feed_forward"] is None and again["layers"][1]["mixer_post_norm"] == j["layers"][1]["mixer_post_norm"]


def broken(path, value):
    d = copy.deepcopy(CASE_A)
    node = d
    for k in path[:-1]:
        node = node[k]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return d


@pytest.mark.parametrize("path,value,needle", [
    (["vocab"], KeyError, "vocab"), (["width"], 0, "positive"), (["norm", "eps"], 0.0, "eps"), (["norm"], KeyError, "norm"),
    (["layers", 0, "type"], "conv", "not known"), (["layers", 1, "mixer", "left"], KeyError, "left"),
    (["layers", 1, "mixer", "left", "rot", "dims"], 7, "dims"), (["layers", 1, "mixer", "left", "rot", "dims"], 26, "dims"),
    (["layers", 1, "mixer", "left", "kv_heads"], 3, "multiple"), (["layers", 3, "mixer", "left", "mask", "size"], 0, "size"),
    (["layers", 1, "mixer", "right", "groups"], 2, "multiple"), (["layers", 1, "mixer", "right", "norm_groups"], 5, "norm_groups"),
    (["layers", 1, "mixer", "right", "state"], KeyError, "state"), (["layers", 1, "mixer", "right", "conv"], 0, "conv"),
    (["layers", 3, "mixer", "right", "kv_heads"], 3, "multiple"), (["layers", 3, "mixer", "right", "dim"], KeyError, "dim"),
    (["layers", 0, "mixer", "rot_dim"], 7, "rot_dim"), (["layers", 0, "mixer", "rot", "dims"], 4, "rot_dim"),
    (["layers", 0, "mixer", "kv_rank"], KeyError, "kv_rank"), (["layers", 2, "mixer", "kv_from"], 2, "earlier"),
    (["layers", 2, "mixer", "kv_from"], 1, "no latent"), (["layers", 2, "mixer", "kv_rank"], 24, "must equal"),
    (["layers", 2, "mixer", "rot", "base"], 500.0, "must equal"), (["layers", 0, "mlp", "kind"], "moe", "not known"),
    (["layers", 0, "mlp", "ff"], 0, "ff"), (["layers"], [], "layers"),
])
def test_what_the_reader_refuses(path, value, needle):
    from fastgguf_b200.config import ConfigError
    from fastgguf_b200.registry import config_from_dict
    with pytest.raises(ConfigError) as e:
        config_from_dict(broken(path, value))
    assert needle in str(e.value)


def test_a_scaling_with_wrong_bands_is_refused():
    from fastgguf_b200.config import ConfigError
    from fastgguf_b200.registry import config_from_dict
    d = copy.deepcopy(CASE_B)
    d["layers"][1]["mixer"]["left"]["rot"]["scaling"]["high"] = 1.0
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert "high" in str(e.value)


def test_weights_are_checked_against_the_configuration(tmp_path):
    from fastgguf_b200.registry import config_from_dict
    from fastgguf_b200.weights import WeightError, check_weights, expected_tensors
    for name, cfg in CASES.items():
        declared = expected_tensors(config_from_dict(cfg))
        want = tensor_shapes(cfg)
        assert sorted(declared) == sorted(want), name
        for k, v in declared.items():
            assert tuple(v["shape"]) == tuple(want[k]), (name, k)
    W = random_weights(CASE_A, 1)
    good = write_model(tmp_path / "good", CASE_A, W)
    assert len(check_weights(config_from_dict(CASE_A), model_dir=good)) == len(W)
    bad = dict(W)
    del bad["l3.mix.left.sink"]
    bad["l2.mlp.up"] = W["l0.mlp.up"]                 # a layer without a feed-forward has no tensors for one
    bad["l2.mix.dkv"] = W["l0.mix.dkv"]               # a layer that reads another's latents has no map of its own
    bad["l1.mix.left.g"] = W["l1.mix.left.g"][:4].contiguous()      # a gate per head where the design has one per number
    with pytest.raises(WeightError) as e:
        check_weights(config_from_dict(CASE_A), model_dir=write_model(tmp_path / "bad", CASE_A, bad))
    assert e.value.missing == ["l3.mix.left.sink"] and e.value.unexpected == ["l2.mix.dkv", "l2.mlp.up"] and "l1.mix.left.g" in e.value.wrong[0]


def test_random_model_folder(tmp_path):
    """The framework's own writer of seeded random folders makes a folder that its reader accepts."""
    from fastgguf_b200.registry import config_from_dict, config_from_dir
    from fastgguf_b200.weights import check_weights, write_random_model
    d = write_random_model(config_from_dict(CASE_C), 5, str(tmp_path / "r"))
    again = config_from_dir(d)
    assert again.describe()["layer_kinds"] == config_from_dict(CASE_C).describe()["layer_kinds"]
    assert len(check_weights(again, model_dir=d)) == len(tensor_shapes(CASE_C))


def test_kernel_libraries_by_model():
    from fastgguf_b200 import capi
    from fastgguf_b200.registry import config_from_dict
    spec = config_from_dict(CASE_B).spec_json()           # no head of 64 or 128 numbers anywhere: no tensor-core attention
    assert capi.kernel_modules_for(spec, capi.FG_BF16) == ("core", "tc", "mix")
    assert capi.kernel_modules_for(spec, capi.FG_F32) == ("core", "mix")
    spec = config_from_dict(CASE_C).spec_json()           # the left side of a pair has heads of 64
    assert capi.kernel_modules_for(spec, capi.FG_BF16) == ("core", "tc", "attn", "mix")
