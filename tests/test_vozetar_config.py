"""Vozetar on the host: from config.json to the plan, the tensor table and a random-weights folder.  No GPU needed."""
import copy

import pytest

import vozetar_configs as C


def test_the_architecture_is_registered():
    import velomind_b200 as vm
    assert "Vozetar" in vm.registered_architectures()
    d = vm.describe_config(C.config("a"))
    assert d["architecture"] == "Vozetar" and d["hidden_size"] == 88 and d["vocab_size"] == 150 and d["max_positions"] == 0
    assert d["runs"] == 4 and len(d["blocks"]) == 4


def test_tensor_table_follows_the_layer_list():
    import velomind_b200 as vm
    t = {k: v["shape"] for k, v in vm.weight_table(C.config("a")).items()}
    assert t["embed"] == [150, 88] and t["bigram"] == [62, 88] and t["head"] == [150, 88] and t["final.norm"] == [88]
    # two mixers side by side: attention with biases and a sink, retention without either
    assert t["l0.mix.left.q"] == [60, 88] and t["l0.mix.left.q.b"] == [60] and t["l0.mix.left.k"] == [20, 88] and t["l0.mix.left.v"] == [12, 88]
    assert t["l0.mix.left.sink"] == [3] and t["l0.mix.left.o"] == [88, 36] and "l0.mix.left.o.b" not in t and "l0.mix.left.g" not in t
    assert t["l0.mix.right.q"] == [24, 88] and t["l0.mix.right.v"] == [20, 88] and t["l0.mix.right.g"] == [20, 88] and t["l0.mix.right.o"] == [88, 20]
    assert "l0.mix.right.norm" not in t and "l0.mix.right.q.b" not in t and "l0.mix.left.out" not in t
    # the wiring's numbers: one set per sublayer
    assert t["l0.hc1.in"] == [3] and t["l0.hc1.out"] == [3] and t["l0.hc1.mix"] == [3, 3] and t["l0.hc2.mix"] == [3, 3]
    assert t["l0.mlp.router"] == [6, 88] and t["l0.mlp.e5.gate"] == [24, 88] and t["l0.mlp.shared.down"] == [88, 40] and "l0.mlp.router.b" not in t
    # attention with a convolution on q, k and v, biases also on the output, a gate per value; no feed-forward: no second norm or wiring
    assert t["l1.mix.q.conv"] == [40, 3] and t["l1.mix.k.conv"] == [20, 3] and t["l1.mix.v.conv"] == [28, 3] and t["l1.mix.o.b"] == [88]
    assert t["l1.mix.g"] == [56, 88] and t["l1.mix.sink"] == [4] and "l1.norm2" not in t and "l1.hc2.in" not in t
    # values that are the keys: no value matrix; norms over the whole projections; a gate per head; the decay's low-rank pair
    assert "l2.mix.left.v" not in t and t["l2.mix.left.q.norm"] == [24] and t["l2.mix.left.k.norm"] == [24] and t["l2.mix.left.g"] == [2, 88]
    assert t["l2.mix.left.q.conv"] == [24, 2] and "l2.mix.left.sink" not in t and "l2.mix.left.q.b" not in t
    assert t["l2.mix.right.a1"] == [7, 88] and t["l2.mix.right.a2"] == [18, 7] and t["l2.mix.right.a2.b"] == [18] and t["l2.mix.right.norm"] == [10]
    assert t["l2.mix.left.out"] == [88] and t["l2.mix.right.out"] == [88]
    assert t["l2.mlp.gate"] == [72, 88] and t["l2.mlp.down"] == [88, 72]
    assert "l3.mlp.shared.up" not in t


def test_the_decay_rank_comes_from_the_checkpoint():
    import velomind_b200 as vm
    cfg = C.config("a")
    del cfg["layers"][2]["mixer"]["right"]["decay_rank"]
    cfg["tensor_shapes"] = {"l2.mix.right.a1": [11, 88]}
    assert vm.weight_table(cfg)["l2.mix.right.a2"]["shape"] == [18, 11]


def test_without_streams_and_without_the_second_table():
    import velomind_b200 as vm
    t = vm.weight_table(C.config("d"))
    assert "bigram" not in t and not any(".hc" in k for k in t) and t["embed"]["shape"] == [96, 64]
    assert t["l0.norm2"]["shape"] == [64] and "l1.norm2" not in t


@pytest.mark.parametrize("damage,word", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("left"), "left"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.9]), "decays"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.9, 1.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=12), "rot"),
    (lambda c: c["layers"][2]["mixer"]["right"].pop("tau"), "tau"),
    (lambda c: c["layers"][2]["mixer"]["left"].update(vdim=10), "vdim"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["embedding"]["bigram"].pop("buckets"), "buckets"),
    (lambda c: c.update(streams=17), "streams"),
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
    for which in ("a", "b", "c", "d"):
        folder = vm.write_random_model(str(tmp_path / which), C.config(which), seed=1)
        vm.check_model_folder(folder)
        assert set(vm.safetensors_info(folder + "/model.safetensors")) == set(vm.weight_table(C.config(which)))
