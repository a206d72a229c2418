"""The Pirozen configuration on the host, without a GPU: reading config.json, what it refuses, the model spec it becomes
(two norms a layer, the token input, the loop as a schedule), and the check of a checkpoint against it."""
import copy

import pytest

from pirozen_cases import CASES, CASE_A, CASE_B, CASE_C, CASE_D, random_weights, tensor_shapes, write_model


def test_registered_and_chosen_by_name():
    from fastgguf_b200.config import PirozenConfig
    from fastgguf_b200.registry import config_from_dict, registered_architectures
    assert "Pirozen" in registered_architectures()
    cfg = config_from_dict(CASE_A)
    assert isinstance(cfg, PirozenConfig) and cfg.architecture == "Pirozen"
    assert cfg.to_dict() == CASE_A
    d = cfg.describe()
    assert d["hidden_size"] == 96 and d["vocab_size"] == 211 and d["num_hidden_layers"] == 4 and d["layer_runs"] == 8
    assert d["layer_kinds"] == ["attention+moe", "attention+moe", "attention+none", "attention+moe"]
    # keys and values of every RUN of a layer: the span in the middle runs three times with caches of its own
    assert d["kv_bytes_per_token"]["bfloat16"] == 2 * (2 * (24 + 40) + 3 * 3 * (16 + 16) + 3 * 1 * (32 + 8) + 2 * (16 + 24))
    assert d["state_bytes_per_sequence"] == 0
    n = sum(a * b if len(s) == 2 else s[0] for s in tensor_shapes(CASE_A).values() for a, b in [s if len(s) == 2 else (s[0], 1)])
    assert d["parameters"] == n


def test_the_loop_becomes_a_schedule():
    from fastgguf_b200.registry import config_from_dict
    spec = config_from_dict(CASE_A).spec_json()
    assert [(r["layer"], r.get("reenter", False)) for r in spec["schedule"]] == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True),
                                                                     (2, False), (3, False)]
    assert spec["reentry"]["kind"] == "concat_linear" and spec["reentry"]["tensors"] == {"weight": "loop.in"}
    once = config_from_dict(CASE_D).spec_json()
    assert [(r["layer"], r.get("reenter", False)) for r in once["schedule"]] == [(0, False), (1, True)]
    both = config_from_dict(CASE_C).spec_json()
    assert [(r["layer"], r.get("reenter", False)) for r in both["schedule"]] == [(0, True), (1, False), (0, True), (1, False)]
    none = config_from_dict(CASE_B).spec_json()
    assert "reentry" not in none and [r["layer"] for r in none["schedule"]] == [0, 1, 2, 3] and not any("reenter" in r for r in none["schedule"])


def test_spec_follows_the_file():
    from fastgguf_b200.registry import config_from_dict
    spec = config_from_dict(CASE_A).spec_json()
    kinds = [(l["block"], l["mixer"]["kind"], (l["feed_forward"] or {}).get("kind")) for l in spec["layers"]]
    assert kinds == [("parallel", "sink_attention", "moe"), ("parallel", "sink_attention", "moe"), ("parallel", "sink_attention", None),
                     ("parallel", "sink_attention", "moe")]
    # two norms where there is a feed-forward, one where there is none
    assert [l.get("feed_forward_norm") is not None for l in spec["layers"]] == [True, True, False, True]
    assert spec["layers"][0]["feed_forward_norm"]["tensors"] == {"weight": "l0.norm2"} and spec["layers"][0]["mixer_norm"]["tensors"] == {"weight": "l0.norm1"}
    a = spec["layers"][0]["mixer"]["params"]
    assert (a["window"], a["n_heads"], a["n_kv_heads"], a["head_dim"], a["v_head_dim"], a["scale"], a["eps"]) == (9, 4, 2, 24, 40, 0.3, 1e-6)
    assert a["bias"] and a["o_bias"] and a["qk_norm"] == "head" and a["gate"] == "head" and not a.get("sink")
    assert a["position"]["params"] == {"head_dim": 24, "theta": 10000.0, "rotary_dim": 8, "layout": "halves",
                                       "scaling": {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64.0, "beta_fast": 8.0,
                                                   "beta_slow": 1.0}}
    assert spec["layers"][1]["mixer"]["params"]["position"]["params"]["scaling"] is None
    p = spec["layers"][2]["mixer"]["params"]
    assert p["window"] == 0 and p["position"] is None
    f = spec["layers"][0]["feed_forward"]["params"]
    assert (f["router"], f["d_ff"], f["n_experts"], f["top_k"], f["n_identity"], f["n_groups"], f["keep_groups"], f["route_scale"], f["shared_d_ff"]) == \
        ("softmax_grouped", 40, 6, 2, 2, 2, 1, 2.0, 56)
    # what the file leaves out the model does not have: no identity experts, one group, no shared expert, weights as they are
    g = spec["layers"][1]["feed_forward"]["params"]
    assert (g["n_experts"], g["top_k"], g["n_identity"], g["n_groups"], g["keep_groups"], g["route_scale"], g["shared_d_ff"]) == (5, 3, 0, 1, 1, 1.0, 0)
    assert not any(k.startswith("shared.") for k in spec["layers"][1]["feed_forward"]["tensors"])
    # every layer reads its own columns of the one table, in a loop too
    t = [l["token_input"]["params"] for l in spec["layers"]]
    assert [(x["column"], x["dim"], x["table_dim"]) for x in t] == [(0, 8, 32), (8, 8, 32), (16, 8, 32), (24, 8, 32)]
    assert spec["layers"][3]["token_input"]["tensors"] == {"table": "side.embed", "gate": "l3.side.gate", "proj": "l3.side.proj", "norm": "l3.side.norm"}
    assert all(l.get("token_input") is None for l in config_from_dict(CASE_B).spec_json()["layers"])
    assert spec["head"]["tensors"]["weight"] == "head" and spec["embedding"]["tensors"]["weight"] == "embed"


def test_python_spec_round_trip():
    from fastgguf_b200.engine.spec import ModelSpec
    from fastgguf_b200.registry import config_from_dict
    j = config_from_dict(CASE_A).spec_json()
    again = ModelSpec.from_json(j).to_json()
    assert again["schedule"] == j["schedule"] and again["reentry"] == j["reentry"]
    assert again["layers"][2]["feed_forward"] is None and again["layers"][2].get("feed_forward_norm") is None
    assert again["layers"][1]["token_input"] == j["layers"][1]["token_input"]
    assert again["layers"][0]["feed_forward_norm"] == j["layers"][0]["feed_forward_norm"]


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
    (["layers", 0, "type"], "conv", "not known"), (["layers", 0, "mixer", "heads"], 0, "positive"),
    (["layers", 0, "mixer", "rot", "dims"], 7, "dims"), (["layers", 0, "mixer", "rot", "dims"], 26, "dims"),
    (["layers", 0, "mixer", "kv_heads"], 3, "multiple"), (["layers", 0, "mixer", "mask", "size"], 0, "size"),
    (["layers", 0, "mixer", "rot", "scaling", "factor"], 0.0, "positive"), (["layers", 0, "mixer", "rot", "base"], 1.0, "base"),
    (["layers", 0, "mlp", "kind"], "dense", "not known"), (["layers", 0, "mlp", "expert", "ff"], 0, "positive"),
    (["layers", 0, "mlp", "router", "top"], 5, "top"), (["layers", 0, "mlp", "router", "groups", "count"], 3, "groups"),
    (["layers", 0, "mlp", "router", "groups", "keep"], 3, "keep"), (["layers", 0, "mlp", "router"], KeyError, "router"),
    (["token_side", "dim"], 0, "dim"), (["loop", "stop"], 5, "stop"), (["loop", "start"], 3, "start"), (["loop", "times"], 0, "times"),
    (["layers"], [], "layers"),
])
def test_what_the_reader_refuses(path, value, needle):
    from fastgguf_b200.config import ConfigError
    from fastgguf_b200.registry import config_from_dict
    with pytest.raises(ConfigError) as e:
        config_from_dict(broken(path, value))
    assert needle in str(e.value)


def test_weights_are_checked_against_the_configuration(tmp_path):
    from fastgguf_b200.registry import config_from_dict
    from fastgguf_b200.weights import WeightError, check_weights, expected_tensors
    for name, case in CASES.items():
        declared = expected_tensors(config_from_dict(case))
        want = tensor_shapes(case)
        assert sorted(declared) == sorted(want), name
        for k, v in declared.items():
            assert tuple(v["shape"]) == tuple(want[k]), (name, k)
    W = random_weights(CASE_A, 1)
    good = write_model(tmp_path / "good", CASE_A, W)
    assert len(check_weights(config_from_dict(CASE_A), model_dir=good)) == len(W)
    bad = dict(W)
    del bad["l1.mix.o.b"]
    bad["l2.mlp.router"] = W["l0.mlp.router"]            # a layer without a feed-forward has no tensors for one
    bad["l3.mlp.e8.up"] = W["l3.mlp.e8.up"][:, :-1].contiguous()
    bad["l0.mix.q.norm"] = W["l0.mix.q.norm"].repeat(4)  # one weight vector for all heads, not one a head
    with pytest.raises(WeightError) as e:
        check_weights(config_from_dict(CASE_A), model_dir=write_model(tmp_path / "bad", CASE_A, bad))
    assert e.value.missing == ["l1.mix.o.b"] and e.value.unexpected == ["l2.mlp.router"]
    assert len(e.value.wrong) == 2 and all(any(n in w for w in e.value.wrong) for n in ("l0.mix.q.norm", "l3.mlp.e8.up"))


def test_random_model_folder(tmp_path):
    """The framework's own writer of seeded random folders gives a folder the reader and the weight check accept."""
    from fastgguf_b200.registry import config_from_dict, config_from_dir
    from fastgguf_b200.weights import check_weights, write_random_model
    d = write_random_model(config_from_dict(CASE_C), 5, str(tmp_path / "r"))
    again = config_from_dir(d)
    assert again.describe()["layer_kinds"] == ["attention+moe", "attention+moe"] and {k: v for k, v in again.to_dict().items() if k != "torch_dtype"} == CASE_C
    assert len(check_weights(again, model_dir=d)) == len(tensor_shapes(CASE_C))


def test_kernel_libraries_by_model():
    from fastgguf_b200 import capi
    from fastgguf_b200.registry import config_from_dict
    spec = config_from_dict(CASE_A).spec_json()
    assert capi.kernel_modules_for(spec, capi.FG_BF16) == ("core", "tc", "mix")
    assert capi.kernel_modules_for(spec, capi.FG_F32) == ("core", "mix")
    # heads of 64 or 128 numbers for keys and values alike: the tensor-core attention kernels as well
    assert capi.kernel_modules_for(config_from_dict(CASE_B).spec_json(), capi.FG_BF16) == ("core", "tc", "attn", "mix")
