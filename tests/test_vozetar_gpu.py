"""The Vozetar design in the library against the plain implementation (tests/plain_vozetar.py): each mechanism alone (through the
probe architecture of the tests' plug-in, which lets one part's output reach the logits), whole models cut into steps in several ways,
weights shaped so that a fault would show where random ones would hide it, and generation through the entry points."""
import copy
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_vozetar as P
import schedules as S
import vozetar_configs as C
from test_kogilix_gpu import (ff_block, mixer_block, probe_config, random_tensors, rounded_to_bf16, run_cuts, standard_cuts, steps_in_pieces,
                              write_model)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MIX, FF = "layers.0.mixer.", "layers.0.feed_forward."
EPS = 1e-5


# ----------------------------------------------------------------------------- a part's arguments, and the same as a configuration
def rotary(kind, dim, base, dims):
    return {"kind": kind, "args": {"head_dim": dim, "theta": base, "rotary_dim": dims}}


def attention_args(hidden, m, form):
    """The arguments of `general_attention` for one of the design's three forms of softmax attention; m as the configuration has it."""
    a = {"hidden": hidden, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"], "eps": EPS,
         "taps": m.get("conv", 0),
         "position": rotary("rotary_half_split" if form == "full" else "rotary_interleaved", m["dim"], m["rot"]["base"], m["rot"]["dims"])}
    if "mask" in m:
        a.update(window=m["mask"]["size"], keep_first=m["mask"]["keep_first"])
    a.update({"full": {"bias": 1, "out_bias": 1, "sink": 1, "gate": "values"}, "window": {"bias": 1, "sink": 1},
              "keys": {"values_are_keys": 1, "qk_norm": 1, "gate": "heads"}}[form])
    return a


def retention_args(hidden, m):
    return {"hidden": hidden, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "decay": "fixed", "decays": list(m["decay"]),
            "k_scale": m["dim"] ** -0.5, "eps": EPS, "position": rotary("rotary_half_split", m["dim"], m["rot"]["base"], m["rot"]["dims"])}


def gated_memory_args(hidden, m):
    return {"hidden": hidden, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "decay": "channel", "tau": m["tau"], "decay_rank": m["decay_rank"],
            "q_scale": m["dim"] ** -0.5, "norm_weight": 1, "eps": EPS}


def side_args(hidden, m, kind):
    if kind == "parallel":
        return {"hidden": hidden, "join": "weighted", "left_scale": m["left_scale"], "right_scale": m["right_scale"],
                "left": {"kind": "general_attention", "args": attention_args(hidden, m["left"], "window")},
                "right": {"kind": "decayed_memory", "args": retention_args(hidden, m["right"])}}
    return {"hidden": hidden, "join": "normed_mean", "eps": EPS,
            "left": {"kind": "general_attention", "args": attention_args(hidden, m["left"], "keys")},
            "right": {"kind": "decayed_memory", "args": gated_memory_args(hidden, m["right"])}}


def moe_args(hidden, mlp):
    a = {"hidden": hidden, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "ff": mlp["expert"]["ff"], "routing": "sigmoid", "glu": 3,
         "activation": "silu"}
    if mlp["router"].get("groups"):
        a.update(groups=mlp["router"]["groups"]["count"], groups_keep=mlp["router"]["groups"]["keep"], groups_top=2)
    if mlp.get("shared"):
        a.update(shared_ff=mlp["shared"]["ff"], shared_gate=0)
    return a


# name -> (role, part kind, hidden, the configuration's own object, form)
MECHANISMS = {
    # every earlier token; three taps; grouped keys (4 on 2); a rotation over 6 of 10 values; sizes that are no multiple of 8
    "attention_full": ("mixer", "general_attention", 56, C.attention(4, 2, 10, 14, 0.45, 3, base=50.0, dims=6), "full"),
    # sizes the tensor-core kernel of prompts takes (bfloat16): heads of 64, four taps
    "attention_full_tiles": ("mixer", "general_attention", 128, C.attention(4, 2, 64, 64, 0.125, 4, base=10000.0), "full"),
    # one tap: the convolution is a scale per channel and keeps nothing
    "attention_one_tap": ("mixer", "general_attention", 64, C.attention(2, 1, 16, 24, 0.3, 1), "full"),
    # a window that ends inside a page with five kept tokens; one key head for three query heads
    "attention_window": ("mixer", "general_attention", 80, C.windowed(3, 1, 24, 8, 0.3, 50, 5, base=500.0, dims=8), "window"),
    # a window of exactly one page, more kept tokens than one page's first chunk of 32
    "attention_window_tiles": ("mixer", "general_attention", 128, C.windowed(4, 2, 32, 32, 0.2, 64, 40, base=200000.0, dims=16), "window"),
    # a window over three pages and nothing kept
    "attention_window_far": ("mixer", "general_attention", 64, C.windowed(2, 2, 16, 16, 0.25, 130, 0), "window"),
    # values that are the keys, norms over the whole projections, a gate per head
    "attention_keys": ("mixer", "general_attention", 72, C.windowed(3, 3, 12, 12, 0.4, 37, 2, base=100.0, dims=4, conv=4), "keys"),
    "attention_keys_tiles": ("mixer", "general_attention", 128, C.windowed(4, 2, 64, 64, 0.15, 100, 6, base=1e6, dims=32, conv=2), "keys"),
    "retention": ("mixer", "decayed_memory", 72, C.retention(3, 12, 20, (0.9, 0.97, 0.995), base=1000.0, dims=8), "retention"),
    # keys wider than a warp's band of 64 channels allows in one pass of four; values wider than one block's 32 columns, the last slice ragged
    "retention_wide": ("mixer", "decayed_memory", 64, C.retention(1, 72, 40, (0.98,), dims=72), "retention"),
    "retention_sliced": ("mixer", "decayed_memory", 64, C.retention(2, 18, 80, (1.0, 0.5), dims=2), "retention"),
    "gated_memory": ("mixer", "decayed_memory", 72, C.gated_memory(3, 12, 20, 4.0, 5), "gated"),
    "gated_memory_tau_one": ("mixer", "decayed_memory", 64, C.gated_memory(2, 32, 16, 1.0, 16), "gated"),
    "side_by_side": ("mixer", "side_by_side", 64, {"left": C.windowed(2, 1, 16, 8, 0.3, 40, 3, dims=8), "left_scale": 0.9,
                                                   "right": C.retention(2, 8, 12, (0.95, 0.99), dims=8), "right_scale": 1.4}, "parallel"),
    "side_by_side_normed": ("mixer", "side_by_side", 64, {"left": C.windowed(2, 2, 16, 16, 0.3, 45, 4, dims=8, conv=3),
                                                          "right": C.gated_memory(2, 8, 12, 8.0, 4)}, "parallel_2"),
    "experts_groups": ("feed_forward", "routed_experts", 64, C.moe(8, 3, 24, 40, groups=(4, 2)), "moe"),
    "experts_groups_one_stays": ("feed_forward", "routed_experts", 48, C.moe(9, 2, 16, groups=(3, 1)), "moe"),
    "experts_top_one": ("feed_forward", "routed_experts", 48, C.moe(7, 1, 16), "moe"),
    "experts_all": ("feed_forward", "routed_experts", 48, C.moe(3, 3, 20, 8), "moe"),
}


def part_args(name):
    role, kind, hidden, m, form = MECHANISMS[name]
    if form in ("full", "window", "keys"):
        return attention_args(hidden, m, form)
    if form == "retention":
        return retention_args(hidden, m)
    if form == "gated":
        return gated_memory_args(hidden, m)
    if form in ("parallel", "parallel_2"):
        return side_args(hidden, m, form)
    return moe_args(hidden, m)


def plain_mechanism(name, x, w):
    role, kind, hidden, m, form = MECHANISMS[name]
    sub = P.sub(w, MIX if role == "mixer" else FF)
    if form == "full":
        return P.mixer_attention(x, sub, m, EPS)
    if form == "window":
        o = P.softmax_branch(x, sub, m, EPS, bias=True, taps_on=False, qk_norm=False, pairing="interleaved", sink=True, values_are_keys=False)
        return P.lin(o.reshape(o.shape[0], -1), sub["o"])
    if form == "keys":
        o = P.softmax_branch(x, sub, m, EPS, bias=False, taps_on=True, qk_norm=True, pairing="interleaved", sink=False, values_are_keys=True)
        o = o * P.sigmoid(P.lin(x, sub["g"]))[:, :, None]
        return P.lin(o.reshape(o.shape[0], -1), sub["o"])
    if form == "retention":
        return P.retention_branch(x, sub, m, EPS)
    if form == "gated":
        return P.gated_memory_branch(x, sub, m, EPS)
    if form == "parallel":
        return P.mixer_parallel(x, sub, m, EPS)
    if form == "parallel_2":
        return P.mixer_parallel_2(x, sub, m, EPS)
    return P.routed_unit(x, sub, m)


def shape_weights(w, rng):
    """Random weights that let every branch show: sinks and biases as strong as the scores, strong taps, decay logits that spread,
    router scores that spread."""
    for name in list(w):
        if name.endswith("sink"):
            w[name] = rng.normal(0.5, 1.0, w[name].shape).astype(np.float32)
        elif name.endswith(".conv"):
            w[name] = rng.normal(0.0, 0.6, w[name].shape).astype(np.float32)
        elif name.endswith(".b"):
            w[name] = rng.normal(0.0, 0.5, w[name].shape).astype(np.float32)
        elif name.endswith("a2"):
            w[name] = rng.normal(0.0, 1.5, w[name].shape).astype(np.float32)
        elif name.endswith("router"):
            w[name] = (w[name] * 4.0).astype(np.float32)
    return w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name, dtype, toy_plugin, tmp_path):
    import velomind_b200 as vm
    role, kind, hidden, m, form = MECHANISMS[name]
    args = part_args(name)
    cfg = probe_config(hidden, mixer_block(kind, args) if role == "mixer" else ff_block(kind, args))
    rng = np.random.default_rng(sum(name.encode()))
    w = shape_weights(random_tensors(vm.weight_table(cfg), rng, 0.25), rng)
    if dtype == "bfloat16":
        w = rounded_to_bf16(w)              # stored as bfloat16; the plain implementation runs on the same rounded numbers
    folder = write_model(str(tmp_path / name), cfg, w, as_bf16=dtype == "bfloat16")
    engine = vm.Engine(vm.load_model(folder, dtype, "cuda:0"), 64 * 6, max_slots=3)      # few pages and slots: both are used again
    requests = S.make_requests(hidden, (70, 5, 130, 64, 1, 65), seed=3)
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        plain[rid] = x + plain_mechanism(name, x, w)
    if form == "moe":                       # the test sees a wrong expert only if the routing spreads, and a wrong group only if groups differ
        x = w["embed.weight"].astype(np.float64)
        scores = P.sigmoid(P.lin(x, w[FF + "router"]))
        picks = [tuple(P.choose_experts(s, m["router"]["top"], m["router"].get("groups"))) for s in scores]
        assert len({e for p in picks for e in p}) == m["router"]["experts"]
        if m["router"].get("groups"):
            assert any(tuple(P.choose_experts(s, m["router"]["top"], None)) != p for s, p in zip(scores, picks))
    cuts = standard_cuts(requests)
    cuts["pieces"] = steps_in_pieces(requests, (2, 3, 64, 1, 65))
    run_cuts(engine, requests, plain, cuts, 3e-5 if dtype == "float32" else 2.5e-2)


# ----------------------------------------------------------------------------- the wiring over several copies of the stream
def streams_config(hidden, streams, with_ff=True):
    ident = {"kind": "identity", "args": {"size": hidden}}
    norm = {"kind": "rmsnorm", "args": {"size": hidden, "eps": EPS}}
    mixer = {"kind": "decayed_memory", "args": retention_args(hidden, C.retention(2, 8, 8, (0.9, 0.99), dims=8))}
    ff = {"kind": "gated", "args": {"hidden": hidden, "intermediate": 40, "activation": "silu", "gate": "gate", "up": "up", "down": "down"}}
    block = {"arrangement": "hyper_connections", "arrangement_args": {"hidden": hidden, "streams": streams, "feed_forward": 1 if with_ff else 0},
             "mixer": mixer, "feed_forward": ff if with_ff else {"kind": "none"}, "mixer_norm": norm,
             "feed_forward_norm": norm if with_ff else {"kind": "none", "args": {}}}
    return {"architectures": ["ProbeForCausalLM"], "hidden": hidden, "vocab": hidden, "limit": 4096, "streams": streams,
            "embedding": {"kind": "token_table", "args": {"vocab": hidden, "hidden": hidden}}, "final_norm": ident, "head": ident,
            "blocks": [block, copy.deepcopy(block)]}


@pytest.mark.parametrize("streams,with_ff", [(1, True), (2, True), (3, True), (4, False), (8, True), (11, True)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_copies_of_the_stream_are_read_mixed_and_summed(streams, with_ff, dtype, toy_plugin, tmp_path):
    """Two layers, so that a layer's last write is carried out by the next layer and the last one's by the model; mixing numbers of
    every sign; the copies' sum reaches the logits."""
    import velomind_b200 as vm
    hidden = 48
    cfg = streams_config(hidden, streams, with_ff)
    rng = np.random.default_rng(streams)
    w = random_tensors(vm.weight_table(cfg), rng, 0.25)
    for name in w:
        if name.endswith(".mix"):
            w[name] = (np.eye(streams) + rng.normal(0.0, 0.4, (streams, streams))).astype(np.float32)
        if name.endswith(".in") or name.endswith(".out"):
            w[name] = rng.normal(0.3, 0.8, (streams,)).astype(np.float32)
    if dtype == "bfloat16":
        w = rounded_to_bf16(w)
    folder = write_model(str(tmp_path / "streams"), cfg, w, as_bf16=dtype == "bfloat16")
    engine = vm.Engine(vm.load_model(folder, dtype, "cuda:0"), 64 * 6, max_slots=3)
    requests = S.make_requests(hidden, (70, 5, 90, 1), seed=13)
    m = C.retention(2, 8, 8, (0.9, 0.99), dims=8)
    plain = {}
    for rid, toks in requests.items():
        xs = np.repeat(w["embed.weight"].astype(np.float64)[toks][None], streams, axis=0)
        for l in range(2):
            pre = f"layers.{l}."
            xs = P.sublayer_on_streams(xs, w[pre + "hc1.in"], w[pre + "hc1.out"], w[pre + "hc1.mix"], w[pre + "mixer_norm.weight"], EPS,
                                       lambda a: P.retention_branch(a, P.sub(w, pre + "mixer."), m, EPS))
            if with_ff:
                xs = P.sublayer_on_streams(xs, w[pre + "hc2.in"], w[pre + "hc2.out"], w[pre + "hc2.mix"], w[pre + "feed_forward_norm.weight"], EPS,
                                           lambda a: P.gated_unit(a, P.sub(w, pre + "feed_forward.")))
        plain[rid] = xs.sum(axis=0)
    cuts = standard_cuts(requests)
    cuts["pieces"] = steps_in_pieces(requests, (2, 1, 1, 30, 1))
    run_cuts(engine, requests, plain, cuts, 3e-5 if dtype == "float32" else 4e-2)


def test_a_wiring_that_knows_one_stream_is_refused_under_several(toy_plugin, tmp_path):
    import velomind_b200 as vm
    cfg = streams_config(48, 2)
    cfg["blocks"][1]["arrangement"] = "prenorm"
    with pytest.raises(vm.ConfigError):
        vm.weight_table(cfg)


# ----------------------------------------------------------------------------- the embedding with its table of pairs
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(61, 13, 5), (1, 1, 1), (257, 2000000011, 1999999973)])
def test_the_second_table_is_read_by_the_token_before(buckets, mul_prev, mul_cur, toy_plugin, tmp_path):
    """The previous token crosses steps: prompts cut into pieces of one and two tokens, decode steps, batches, slots used again.  One
    table has a single row beside the first token's; one has multipliers whose products do not fit 32 bits."""
    import velomind_b200 as vm
    hidden, rows = 32, buckets
    ident = {"kind": "identity", "args": {"size": hidden}}
    cfg = {"architectures": ["ProbeForCausalLM"], "hidden": hidden, "vocab": hidden, "limit": 4096, "final_norm": ident, "head": ident, "blocks": [],
           "embedding": {"kind": "token_pairs_table", "args": {"vocab": hidden, "hidden": hidden, "tensor": "weight", "pairs_tensor": "pairs",
                                                               "buckets": rows, "mul_prev": mul_prev, "mul_cur": mul_cur}}}
    rng = np.random.default_rng(buckets % 97)
    w = random_tensors(vm.weight_table(cfg), rng, 1.0)
    assert w["embed.pairs"].shape == (rows + 1, hidden)
    folder = write_model(str(tmp_path / "pairs"), cfg, w)
    engine = vm.Engine(vm.load_model(folder, "float32", "cuda:0"), 64 * 6, max_slots=3)
    requests = S.make_requests(hidden, (70, 5, 130, 64, 1, 65), seed=23)
    plain = {rid: P.embed_tokens(toks, w["embed.weight"], w["embed.pairs"], {"buckets": rows, "mul_prev": mul_prev, "mul_cur": mul_cur})
             for rid, toks in requests.items()}
    cuts = standard_cuts(requests)
    cuts["pieces"] = steps_in_pieces(requests, (2, 1, 1, 3, 64))
    run_cuts(engine, requests, plain, cuts, 1e-6)


# ----------------------------------------------------------------------------- shaped: sharp scores, so that one key off shows
def sharp_model(tmp_path, vm, name, m, form, seed):
    """An attention layer alone whose scores are spread wide (a large `scale`): most queries give nearly all their weight to one or two
    keys, so a key wrongly seen or wrongly hidden changes the answer outright."""
    hidden = 64
    args = attention_args(hidden, m, form)
    cfg = probe_config(hidden, mixer_block("general_attention", args))
    rng = np.random.default_rng(seed)
    w = shape_weights(random_tensors(vm.weight_table(cfg), rng, 0.3), rng)
    w = rounded_to_bf16(w)
    return w, {"float32": write_model(str(tmp_path / (name + "32")), cfg, w), "bfloat16": write_model(str(tmp_path / (name + "16")), cfg, w, as_bf16=True)}


def plain_window(x, w, m, form):
    sub = P.sub(w, MIX)
    if form == "window":
        o = P.softmax_branch(x, sub, m, EPS, bias=True, taps_on=False, qk_norm=False, pairing="interleaved", sink=True, values_are_keys=False)
    else:
        o = P.softmax_branch(x, sub, m, EPS, bias=False, taps_on=True, qk_norm=True, pairing="interleaved", sink=False, values_are_keys=True)
        o = o * P.sigmoid(P.lin(x, sub["g"]))[:, :, None]
    return P.lin(o.reshape(o.shape[0], -1), sub["o"])


@pytest.mark.parametrize("form,window,keep", [("window", 64, 6), ("window", 33, 1), ("keys", 100, 40), ("keys", 75, 0)])
def test_keys_at_the_edges_of_window_and_kept_tokens_decide(form, window, keep, toy_plugin, tmp_path):
    """With sharp scores, a window one token longer or shorter, one kept token more or fewer, or a sink left out gives another answer at
    many places (checked on the plain implementation first); the library must give the right one, in prompts, pieces and decode steps."""
    import velomind_b200 as vm
    m = C.windowed(2, 1, 16, 16, 3.0, window, keep, base=100.0, dims=8, conv=3 if form == "keys" else None)
    w, folders = sharp_model(tmp_path, vm, "edge", m, form, 100 + window)
    requests = S.make_requests(64, (330, 150), seed=window)
    plain, moved, places = {}, 0.0, {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        y = plain_window(x, w, m, form)
        plain[rid] = x + y
        for change in ({"size": window + 1, "keep_first": keep}, {"size": window - 1, "keep_first": keep}, {"size": window, "keep_first": keep + 1},
                       {"size": window, "keep_first": max(keep - 1, 0)}):
            if change["size"] < 1 or (change["keep_first"] == keep and change["size"] == window):
                continue
            other = plain_window(x, w, dict(m, mask=change), form)
            far = np.abs(other - y).max(axis=1)
            key = (change["size"], change["keep_first"])
            places[key] = places.get(key, 0) + int((far[window:] > 0.05 * np.abs(y).max()).sum())
            moved = max(moved, float(far.max()))
    assert moved > 0.2 and min(places.values()) >= 1 and sum(places.values()) >= 8, places          # every edge decides somewhere
    for dtype, tol in (("float32", 5e-5), ("bfloat16", 3e-2)):
        engine = vm.Engine(vm.load_model(folders[dtype], dtype, "cuda:0"), 64 * 8, max_slots=2)
        cuts = {"whole": S.steps_whole(requests), "tail": S.steps_tail_one_by_one(requests, tail=120), "batches": S.steps_unequal_batches(requests, tails=(90, 40)),
                "pieces": steps_in_pieces(requests, (70, 2, 64, 1, 33))}
        run_cuts(engine, requests, plain, cuts, tol)


def test_far_keys_decide_where_every_token_is_visible(toy_plugin, tmp_path):
    """The attention without a window, with sharp scores: keys hundreds of tokens back carry much of the weight (checked on the plain
    implementation: hiding everything beyond 128 tokens gives another answer at many places), across page borders, in prompts, pieces and
    200 decode steps, with three taps whose kept rows cross every cut."""
    import velomind_b200 as vm
    m = C.attention(2, 1, 16, 16, 3.0, 3, base=100.0, dims=8)
    w, folders = sharp_model(tmp_path, vm, "far", m, "full", 11)
    requests = S.make_requests(64, (450, 130), seed=21)
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        y = P.mixer_attention(x, P.sub(w, MIX), m, EPS)
        plain[rid] = x + y
        if len(toks) > 400:
            near = P.mixer_attention(x, P.sub(w, MIX), dict(m, mask={"size": 128, "keep_first": 0}), EPS)
            assert (np.abs(near - y).max(axis=1)[200:] > 0.05 * np.abs(y).max()).sum() >= 20
    for dtype, tol in (("float32", 5e-5), ("bfloat16", 3e-2)):
        engine = vm.Engine(vm.load_model(folders[dtype], dtype, "cuda:0"), 64 * 10, max_slots=2)
        cuts = {"whole": S.steps_whole(requests), "tail": S.steps_tail_one_by_one(requests, tail=200),
                "batches": S.steps_unequal_batches(requests, tails=(150, 60)), "pieces": steps_in_pieces(requests, (70, 2, 64, 1, 129))}
        run_cuts(engine, requests, plain, cuts, tol)


def test_a_sink_left_out_would_show(toy_plugin, tmp_path):
    import velomind_b200 as vm
    m = C.windowed(2, 2, 16, 16, 1.0, 40, 2, dims=8)
    w, folders = sharp_model(tmp_path, vm, "sink", m, "window", 7)
    w[MIX + "sink"] = np.array([3.0, 5.0], np.float32)          # as large as the largest scores: the sink takes a good part of the weight
    folder = write_model(str(tmp_path / "sink"), probe_config(64, mixer_block("general_attention", attention_args(64, m, "window"))), w)
    requests = S.make_requests(64, (90, 20), seed=5)
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        y = plain_window(x, w, m, "window")
        without = dict(w)
        without[MIX + "sink"] = np.array([-60.0, -60.0], np.float32)
        assert np.abs(plain_window(x, without, m, "window") - y).max() > 0.2 * np.abs(y).max()
        plain[rid] = x + y
    engine = vm.Engine(vm.load_model(folder, "float32", "cuda:0"), 64 * 6, max_slots=2)
    run_cuts(engine, requests, plain, standard_cuts(requests), 5e-5)


@pytest.mark.parametrize("form", ["retention", "gated"])
def test_the_memory_is_carried_far(form, toy_plugin, tmp_path):
    """Decays close to 1: what the first tokens wrote still decides the answer hundreds of tokens later (checked on the plain
    implementation: other first tokens, another last row), through a prompt in pieces and 300 decode steps."""
    import velomind_b200 as vm
    hidden = 64
    if form == "retention":
        m = C.retention(2, 16, 16, (0.999, 0.9995), dims=16)
        args = retention_args(hidden, m)
    else:
        m = C.gated_memory(2, 16, 16, 64.0, 4)
        args = gated_memory_args(hidden, m)
    cfg = probe_config(hidden, mixer_block("decayed_memory", args))
    rng = np.random.default_rng(41)
    w = random_tensors(vm.weight_table(cfg), rng, 0.3)
    if form == "gated":
        w[MIX + "a2.b"] = np.full_like(w[MIX + "a2.b"], 3.0)      # decays of sigmoid(3)^(1/64): a memory hundreds of tokens long
    folder = write_model(str(tmp_path / "far"), cfg, w)
    requests = S.make_requests(hidden, (420, 35), seed=6)
    fn = P.retention_branch if form == "retention" else P.gated_memory_branch
    plain = {}
    for rid, toks in requests.items():
        x = w["embed.weight"].astype(np.float64)[toks]
        y = fn(x, P.sub(w, MIX), m, EPS)
        plain[rid] = x + y
        if len(toks) > 400:
            other = list(toks)
            other[:20] = [(t + 7) % hidden for t in toks[:20]]
            y2 = fn(w["embed.weight"].astype(np.float64)[other], P.sub(w, MIX), m, EPS)
            assert np.abs(y2[-1] - y[-1]).max() > 0.02 * np.abs(y).max()
    engine = vm.Engine(vm.load_model(folder, "float32", "cuda:0"), 64 * 8, max_slots=2)
    cuts = {"whole": S.steps_whole(requests), "tail": S.steps_tail_one_by_one(requests, tail=300), "pieces": steps_in_pieces(requests, (100, 2, 64, 1, 7))}
    run_cuts(engine, requests, plain, cuts, 5e-5)


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def voz_folders(tmp_path_factory):
    import velomind_b200 as vm
    root = tmp_path_factory.mktemp("vozetar")
    return {k: vm.write_random_model(str(root / k), C.config(k), seed=s, std=0.12, norm_jitter=0.2, dtype="float32")
            for k, s in (("a", 5), ("b", 6), ("c", 7), ("d", 8))}


def plain_logits(folder, requests):
    cfg, w = P.read_model(folder)
    return cfg, {rid: P.forward(cfg, w, toks) for rid, toks in requests.items()}


@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
def test_whole_model_float32(which, voz_folders):
    import velomind_b200 as vm
    engine = vm.Engine(vm.load_model(voz_folders[which], "float32", "cuda:0"), 64 * 7, max_slots=3)     # few pages and slots: both are used again
    vocab = C.config(which)["vocab"]
    requests = S.make_requests(vocab, (50, 6, 140, 64, 2, 129), seed=8)
    cfg, plain = plain_logits(voz_folders[which], requests)
    cuts = standard_cuts(requests)
    cuts["pieces"] = steps_in_pieces(requests, (3, 2, 64, 70, 1))
    run_cuts(engine, requests, plain, cuts, 1e-4)
    engine.cache.check()


def test_whole_model_bfloat16(voz_folders, tmp_path):
    """The serving precision: weights rounded to bfloat16, then compared with the plain implementation on the SAME rounded weights.
    Every routed layer takes ALL its experts here (a token whose candidates lie closer than the rounding of its input would choose another
    expert and differ by more than rounding); the choice itself is left to the float32 tests."""
    import velomind_b200 as vm
    cfg, w = P.read_model(voz_folders["b"])
    for layer in cfg["layers"]:
        if layer["mlp"] and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
            layer["mlp"]["router"].pop("groups", None)
    bits = rounded_to_bf16(w)
    folder = write_model(str(tmp_path / "b16"), cfg, bits, as_bf16=True)
    engine = vm.Engine(vm.load_model(folder, "bfloat16", "cuda:0"), 64 * 16, max_slots=4)
    requests = S.make_requests(cfg["vocab"], (200, 31, 330), seed=9)
    plain = {rid: P.forward(cfg, bits, toks) for rid, toks in requests.items()}
    scale = max(float(np.abs(v).max()) for v in plain.values())
    for steps in (S.steps_whole(requests), S.steps_tail_one_by_one(requests, tail=40), S.steps_unequal_batches(requests, tails=(30, 11, 45))):
        got = S.run_steps_in_process(engine, steps)
        exp = S.expected_rows(steps, requests, plain)
        err = np.concatenate([np.abs(got[k] - exp[k]).max(axis=1) for k in exp]) / scale
        # rounding alone: two to three parts in a hundred of the largest logit at most places (three layers over two copies of the stream)
        assert np.median(err) < 0.035 and err.max() < 0.15, (float(np.median(err)), float(err.max()))


def test_long_decoding_passes_windows_over_decoded_tokens(voz_folders):
    """300 decode steps behind a short prompt: every window of model a (33 and 70 tokens) moves over decoded tokens only, the kept first
    tokens stay, pages that fell out of every window go back, and steps are replayed from graphs."""
    import velomind_b200 as vm
    engine = vm.Engine(vm.load_model(voz_folders["a"], "float32", "cuda:0"), 64 * 8, max_slots=2)
    assert engine.use_graphs
    requests = S.make_requests(150, (310, 40), seed=10)
    cfg, plain = plain_logits(voz_folders["a"], requests)
    run_cuts(engine, requests, plain, {"tail": S.steps_tail_one_by_one(requests, tail=300), "batch": S.steps_unequal_batches(requests, batch=2, tails=(290, 30))}, 1e-4)
    assert engine.graphs_captured > 0


# ----------------------------------------------------------------------------- through the entry points
def greedy(cfg, w, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(P.forward(cfg, w, seq)[-1].argmax()))
    return seq[len(prompt):]


def test_greedy_generation_through_the_entry_point(voz_folders):
    import velomind_b200 as vm
    cfg, w = P.read_model(voz_folders["a"])
    te = vm.load(voz_folders["a"], dtype="float32", max_tokens=2048)
    prompts = [[1, 2, 3, 4, 5], [100, 7], [9] * 70]
    out = te.generate(prompts, temperature=0.0, max_tokens=6, stop_tokens=())
    assert [len(r.tokens) for r in out] == [6, 6, 6]
    for prompt, r in zip(prompts, out):
        seq = list(prompt)
        for tok in r.tokens:
            row = P.forward(cfg, w, seq)[-1]
            assert row[tok] >= row.max() - 1e-4, (seq, tok, int(row.argmax()))
            seq.append(tok)
    # several decode steps queued on the device give the same tokens: the token before each step's one is found on the device
    again = te.generate(prompts, temperature=0.0, max_tokens=6, stop_tokens=(), steps_per_sync=4)
    assert [r.tokens for r in again] == [r.tokens for r in out]


def test_the_console_program_generates(voz_folders):
    cfg, w = P.read_model(voz_folders["d"])
    want = greedy(cfg, w, [5, 6, 7, 8], 5)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "smollm2_chat"), "--model", voz_folders["d"], "--dtype", "float32", "--temp", "0",
                           "--max-tokens", "5", "--prompt-ids", "5,6,7,8"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("Output: ")][0]
    assert line == "Output: " + "".join(f"[{t}]" for t in want)


def test_trace_replay_program(voz_folders, tmp_path):
    requests = S.make_requests(150, (40, 3, 90), seed=12)
    cfg, plain = plain_logits(voz_folders["a"], requests)
    steps = S.steps_unequal_batches(requests, tails=(20, 2, 33))
    out = str(tmp_path / "out")
    for dtype, tol in (("float32", 1e-4), ("bfloat16", None)):
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", voz_folders["a"], "--dtype", dtype, "--out", out,
                               "--max-tokens", str(64 * 6)], input=S.to_jsonl(steps), text=True, capture_output=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
        want = S.expected_rows(steps, requests, plain)
        scale = max(1.0, max(float(np.abs(v).max()) for v in want.values()))
        for step, rows in want.items():
            got = np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
            assert got.shape == rows.shape
            if tol is not None:
                assert float(np.abs(got - rows).max()) <= tol * scale, step
            else:
                assert np.isfinite(got).all()
