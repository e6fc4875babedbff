"""Fidizen on the host: from config.json to the plan, the tensor table and a random-weights folder.  No GPU needed."""
import copy

import pytest

import fidizen_configs as C


def test_the_architecture_is_registered():
    import velomind_b200 as vm
    assert "Fidizen" in vm.registered_architectures()
    d = vm.describe_config(C.config("a"))
    assert d["architecture"] == "Fidizen" and d["hidden_size"] == 88 and d["vocab_size"] == 150 and d["max_positions"] == 0


def test_tensor_table_follows_the_layer_list():
    import velomind_b200 as vm
    t = {k: v["shape"] for k, v in vm.weight_table(C.config("a")).items()}
    assert t["embed"] == [150, 88] and t["head"] == [150, 88] and t["final.norm"] == [88]
    # queries carry the rotated part head by head, the key/value down-projection carries it once
    assert t["l0.mix.dq"] == [24, 88] and t["l0.mix.dq.norm"] == [24] and t["l0.mix.uq"] == [3 * 26, 24]
    assert t["l0.mix.dkv"] == [42, 88] and t["l0.mix.dkv.norm"] == [36] and t["l0.mix.uk"] == [60, 36] and t["l0.mix.uv"] == [30, 36]
    assert t["l0.mix.sink"] == [3] and t["l0.mix.g"] == [30, 88] and t["l0.mix.o"] == [88, 30]
    assert t["l0.canon1"] == [88, 3] and t["l0.canon2"] == [88, 3] and t["l0.norm1"] == [88] and t["l0.norm2"] == [88]
    # gated experts, a router without a bias, a gated shared expert without a gate of its own
    assert t["l0.mlp.router"] == [5, 88] and "l0.mlp.router.b" not in t and "l0.mlp.correction" not in t
    assert t["l0.mlp.e4.gate"] == [24, 88] and t["l0.mlp.e4.up"] == [24, 88] and t["l0.mlp.e4.down"] == [88, 24] and "l0.mlp.e5.up" not in t
    assert t["l0.mlp.shared.gate"] == [40, 88] and t["l0.mlp.shared.up"] == [40, 88] and t["l0.mlp.shared.down"] == [88, 40]
    assert "l0.mlp.shared.sg" not in t
    # a layer without a feed-forward has neither a second norm nor a second convolution
    assert "l1.norm2" not in t and "l1.canon2" not in t and t["l1.canon1"] == [88, 3] and not any(k.startswith("l1.mlp.") for k in t)
    # layers that run another layer's weights have no tensors
    assert not any(k.startswith("l2.") or k.startswith("l4.") for k in t)
    assert not any(k.startswith("l3.mlp.shared") for k in t)
    assert t["l5.mlp.up"] == [72, 88] and t["l5.mlp.down"] == [88, 72] and t["l5.mlp.act"] == [4]


def test_every_layer_is_a_run_with_a_cache_of_its_own():
    import velomind_b200 as vm
    d = vm.describe_config(C.config("a"))
    assert d["runs"] == 6 and len(d["blocks"]) == 4


def test_one_tap_and_no_taps():
    import velomind_b200 as vm
    t = vm.weight_table(C.config("c"))
    assert t["l0.canon1"]["shape"] == [48, 1]
    cfg = C.config("c")
    del cfg["canon"]
    assert not any("canon" in k for k in vm.weight_table(cfg))


@pytest.mark.parametrize("damage,word", [
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][2].update(weights_of=9), "weights_of"),
    (lambda c: c["layers"][0].update(type="mlstm"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"].pop("rot"), "rot"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=12), "rot"),
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
