"""Semesun on the host: from config.json to the plan, the tensor table and a random-weights folder.  No GPU needed."""
import copy

import pytest

import semesun_configs as C


def test_the_architecture_is_registered():
    import velomind_b200 as vm
    assert "Semesun" in vm.registered_architectures()
    d = vm.describe_config(C.config("a"))
    assert d["architecture"] == "Semesun" and d["hidden_size"] == 96 and d["vocab_size"] == 160 and d["max_positions"] == 0
    assert d["runs"] == 5


def test_tensor_table_follows_the_layer_list():
    import velomind_b200 as vm
    t = {k: v["shape"] for k, v in vm.weight_table(C.config("a")).items()}
    assert t["embed"] == [160, 96] and t["head"] == [160, 96] and t["final.norm"] == [96]
    # a state-space layer: z | x | B | C | dt stacked in one projection, the convolution over x | B | C
    assert t["l0.mix.in"] == [60 + 60 + 24 + 24 + 3, 96] and t["l0.mix.conv"] == [108, 4] and t["l0.mix.conv.b"] == [108]
    assert t["l0.mix.dt_bias"] == [3] and t["l0.mix.A_log"] == [3] and t["l0.mix.D"] == [3] and t["l0.mix.norm"] == [60] and t["l0.mix.o"] == [96, 60]
    assert t["l0.mlp.up"] == [112, 96] and t["l0.mlp.down"] == [96, 112] and "l0.mlp.gate" not in t
    # attention: keys and values of unequal sizes, one norm weight for all heads, a bias table, a blending scalar
    assert t["l1.mix.q"] == [64, 96] and t["l1.mix.k"] == [32, 96] and t["l1.mix.v"] == [48, 96] and t["l1.mix.o"] == [96, 96]
    assert t["l1.mix.q.norm"] == [16] and t["l1.mix.k.norm"] == [16] and t["l1.mix.rel"] == [12, 4] and t["l1.mix.vmix"] == []
    # routed experts: the router also scores the identity experts, which have no tensors
    assert t["l1.mlp.router"] == [9, 96] and t["l1.mlp.correction"] == [9] and "l1.mlp.router.b" not in t
    assert t["l1.mlp.e6.gate"] == [40, 96] and t["l1.mlp.e6.up"] == [40, 96] and t["l1.mlp.e6.down"] == [96, 40] and "l1.mlp.e7.up" not in t
    # a layer that does not blend has no scalar; a layer without a feed-forward has no second norm
    assert "l2.mix.vmix" not in t and t["l2.mix.rel"] == [9, 2] and "l2.norm2" not in t and not any(k.startswith("l2.mlp.") for k in t)
    assert t["l3.mix.vmix"] == [] and t["l4.mix.in"] == [48 + 48 + 20 + 20 + 4, 96] and t["l4.mix.conv"] == [88, 2]


def test_the_first_blending_layer_is_the_source_of_the_others():
    import velomind_b200 as vm
    d = vm.describe_config(C.config("a"))
    roles = [b["mixer"]["args"].get("v_blend") for b in d["blocks"] if b["mixer"]["kind"] == "window_attention"]
    assert roles == ["source", None, "blend"]
    args = d["blocks"][3]["mixer"]["args"]
    assert args["window"] == 70 and args["keep_first"] == 66 and args["bias_rows"] == 20 and args["bias_far"] == 64
    moe = d["blocks"][1]["feed_forward"]["args"]
    assert moe["routing"] == "scored" and moe["groups"] == 3 and moe["groups_keep"] == 2 and moe["identity"] == 2 and moe["glu"] == 1


@pytest.mark.parametrize("damage,word", [
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "v_mix"),                   # values of 16 against the source's 24
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),               # only two of three groups can be chosen from
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][0].update(type="convolution"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mixer"].update(norm_groups=7), "norm_groups"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("bias_max"), "bias_max"),
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


def test_the_rows_of_a_bias_table_come_from_the_checkpoint(tmp_path):
    """config.json does not say how many rows a layer's bias table has: the tensor's shape does."""
    import velomind_b200 as vm
    cfg = C.config("a")
    folder = vm.write_random_model(str(tmp_path / "m"), cfg, seed=2)
    import json
    for layer in cfg["layers"]:
        layer["mixer"].pop("bias_rows", None)
    with open(folder + "/config.json", "w") as f:
        json.dump(cfg, f)
    vm.check_model_folder(folder)        # rows 12, 9 and 20 are found in the file, not the default of 16
