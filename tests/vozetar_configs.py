"""Small Vozetar configurations for the tests.  They differ from one another in every size; head counts, key and value sizes,
windows, kept tokens, tap counts, stream counts and the order of layers are unequal on purpose, and some values that models tend to make
equal or 1 are not (and some are)."""
import copy


def rot(base, dims):
    return {"base": base, "dims": dims}


def attention(heads, kv_heads, dim, vdim, scale, conv, base=10000.0, dims=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "conv": conv, "rot": rot(base, dim if dims is None else dims)}


def windowed(heads, kv_heads, dim, vdim, scale, size, keep_first, base=10000.0, dims=None, conv=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size, "keep_first": keep_first},
         "rot": rot(base, dim if dims is None else dims)}
    if conv is not None:
        m["conv"] = conv
    return m


def retention(heads, dim, vdim, decay, base=10000.0, dims=None):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": rot(base, dim if dims is None else dims)}


def gated_memory(heads, dim, vdim, tau, decay_rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": decay_rank}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared_ff=None, groups=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r, "shared": {"ff": shared_ff} if shared_ff else None}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# Odd sizes that only the plain kernels take; three copies of the stream; windows of 33 and 70 (one inside a page, one across) with 5 and 2
# kept tokens; three and two taps; a rotation over a part of the head; three groups of two experts of which two stay; a layer without a
# feed-forward; grouped keys (3 query heads on 1, 4 on 2).
VOZ_A = {
    "architecture": "Vozetar", "vocab": 150, "width": 88, "streams": 3, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 61, "mul_prev": 13, "mul_cur": 5}},
    "layers": [
        layer("parallel", {"left": windowed(3, 1, 20, 12, 0.21, 33, 5, base=500.0, dims=8), "left_scale": 0.8,
                           "right": retention(2, 12, 10, (0.9, 0.97), base=2000.0, dims=6), "right_scale": 1.3}, moe(6, 2, 24, 40, groups=(3, 2))),
        layer("attention", attention(4, 2, 10, 14, 0.3, 3, base=300.0, dims=6), None),
        layer("parallel_2", {"left": windowed(2, 2, 12, 12, 0.25, 70, 2, base=10000.0, dims=4, conv=2), "right": gated_memory(3, 6, 10, 5.0, 7)}, dense(72)),
        layer("attention", attention(1, 1, 16, 8, 0.2, 2, dims=16), moe(4, 1, 16)),
    ],
}

# Sizes the tensor-core kernels and the vector loads accept (heads of 64 and 32, widths and inner sizes in multiples of 32); two copies of
# the stream; a window of exactly one page and one of 100; four taps; all experts of three; four groups of which one stays.
VOZ_B = {
    "architecture": "Vozetar", "vocab": 320, "width": 256, "streams": 2, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 509, "mul_prev": 33, "mul_cur": 3}},
    "layers": [
        layer("parallel_2", {"left": windowed(4, 2, 64, 64, 0.12, 64, 4, base=1e6, dims=32, conv=4), "right": gated_memory(2, 32, 64, 16.0, 8)}, moe(8, 2, 64, 128, groups=(4, 1))),
        layer("parallel", {"left": windowed(8, 2, 32, 32, 0.18, 100, 1, base=200000.0, dims=16), "left_scale": 1.1,
                           "right": retention(4, 64, 32, (0.96875, 0.99, 0.998, 0.9995), base=1e6, dims=64), "right_scale": 0.6}, dense(384)),
        layer("attention", attention(4, 4, 64, 64, 0.125, 3), moe(3, 3, 128, 64)),
    ],
}

# One copy of the stream (still wired through its in / out / mix numbers), one head, one tap (a convolution that sees nothing but the
# token itself), a window of one token with nothing kept, one group, one expert of two, a decay of exactly 1.
VOZ_C = {
    "architecture": "Vozetar", "vocab": 64, "width": 48, "streams": 1, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 1, "mul_prev": 1, "mul_cur": 1}},
    "layers": [
        layer("attention", attention(1, 1, 24, 40, 0.3, 1, dims=2), dense(40)),
        layer("parallel", {"left": windowed(2, 1, 4, 6, 0.5, 1, 0, dims=4), "left_scale": 1.0,
                           "right": retention(1, 8, 8, (1.0,), dims=8), "right_scale": 1.0}, moe(2, 1, 8, 8, groups=(1, 1))),
        layer("parallel_2", {"left": windowed(1, 1, 8, 8, 0.4, 3, 1, dims=8, conv=1), "right": gated_memory(1, 4, 4, 1.0, 3)}, None),
    ],
}

# No `streams` key and no second table: the plain residual sum around the same mixers.
VOZ_D = {
    "architecture": "Vozetar", "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        layer("parallel", {"left": windowed(2, 2, 16, 16, 0.25, 20, 3, dims=8), "left_scale": 0.7,
                           "right": retention(2, 16, 16, (0.95, 0.99), dims=16), "right_scale": 0.9}, dense(96)),
        layer("attention", attention(2, 1, 16, 16, 0.25, 2), None),
    ],
}


def config(which):
    return copy.deepcopy({"a": VOZ_A, "b": VOZ_B, "c": VOZ_C, "d": VOZ_D}[which])
