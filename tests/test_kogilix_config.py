"""Kogilix on the host: from config.json to the plan, the tensor table and a random-weights folder.  No GPU needed."""
import copy

import pytest

import kogilix_configs as C


def test_the_architecture_is_registered_and_named_by_a_single_key():
    import velomind_b200 as vm
    assert "Kogilix" in vm.registered_architectures()
    d = vm.describe_config(C.config("a"))
    assert d["architecture"] == "Kogilix" and d["hidden_size"] == 96 and d["vocab_size"] == 150 and d["max_positions"] == 0


def test_tensor_table_follows_the_layer_list():
    import velomind_b200 as vm
    t = {k: v["shape"] for k, v in vm.weight_table(C.config("a")).items()}
    assert t["embed"] == [150, 96] and t["head"] == [150, 96] and t["final.norm"] == [96]
    # an mLSTM layer with a dense feed-forward
    assert t["l0.mix.q"] == [48, 96] and t["l0.mix.k"] == [48, 96] and t["l0.mix.v"] == [80, 96] and t["l0.mix.g"] == [80, 96]
    assert t["l0.mix.i"] == [2, 96] and t["l0.mix.f.b"] == [2] and t["l0.mix.norm"] == [80] and t["l0.mix.o"] == [96, 80]
    assert t["l0.mlp.gate"] == [112, 96] and t["l0.mlp.down"] == [96, 112]
    # latent attention with latents of its own, routed experts and a shared expert with its gate
    assert t["l1.mix.dq"] == [48, 96] and t["l1.mix.dq.norm"] == [48] and t["l1.mix.uq"] == [96, 48]
    assert t["l1.mix.dkv"] == [64, 96] and t["l1.mix.dkv.norm"] == [64] and t["l1.mix.uk"] == [96, 64] and t["l1.mix.uv"] == [48, 64]
    assert t["l1.mix.o"] == [96, 48]
    assert t["l1.mlp.router"] == [5, 96] and t["l1.mlp.router.b"] == [5] and t["l1.mlp.e4.up"] == [40, 96] and t["l1.mlp.e4.down"] == [96, 40]
    assert "l1.mlp.e5.up" not in t
    assert t["l1.mlp.shared.up"] == [56, 96] and t["l1.mlp.shared.down"] == [96, 56] and t["l1.mlp.shared.sg"] == [1, 96]
    # a layer on another layer's latents has no down-projection of its own; a layer without a feed-forward has no second norm
    assert "l2.mix.dkv" not in t and "l2.mix.dkv.norm" not in t and t["l2.mix.uk"] == [32, 64] and t["l2.mix.uv"] == [96, 64]
    assert "l2.norm2" not in t and "l2.norm1" in t and not any(k.startswith("l2.mlp.") for k in t)
    # no shared expert
    assert not any(k.startswith("l3.mlp.shared") for k in t) and t["l3.mlp.e3.up"] == [24, 96]


def test_runs_share_a_cache_where_the_configuration_says_so():
    import velomind_b200 as vm
    d = vm.describe_config(C.config("b"))
    assert d["runs"] == 5
    own = [b["mixer"]["args"].get("own_latent", 1) for b in d["blocks"] if b["mixer"]["kind"] == "latent_attention"]
    assert own == [1, 0, 0]


@pytest.mark.parametrize("damage,word", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "kv_from"),              # an mLSTM layer has no latents
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),              # not an earlier layer
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=32), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0].update(type="convolution"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_a_wrong_configuration_is_refused_by_name(damage, word):
    import velomind_b200 as vm
    cfg = copy.deepcopy(C.config("a"))
    damage(cfg)
    with pytest.raises(vm.ConfigError) as e:
        vm.weight_table(cfg)
    assert word in str(e.value)


def test_random_weights_folder_matches_the_model(tmp_path):
    import velomind_b200 as vm
    for which in ("a", "b", "c"):
        folder = vm.write_random_model(str(tmp_path / which), C.config(which), seed=1)
        vm.check_model_folder(folder)
        assert set(vm.safetensors_info(folder + "/model.safetensors")) == set(vm.weight_table(C.config(which)))
