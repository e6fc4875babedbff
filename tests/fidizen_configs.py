"""Small Fidizen configurations for the tests.  They differ from one another in every size; head counts, key, rotated and value
sizes, ranks, windows and tap counts are unequal on purpose, and some values that models tend to make equal or 1 are not
(and some are)."""
import copy


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, base=10000.0, dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if window:
        m["mask"] = {"size": window}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared_ff=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    m["shared"] = {"ff": shared_ff} if shared_ff else None
    return m


def layer(mixer, mlp, weights_of=None):
    out = {"type": "latent_attention", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


# Odd sizes that only the plain kernels take; three taps; windows of 33 and 70 (one inside a page, one across); a layer without
# a feed-forward; two experts of five; a layer run twice more with a cache and state of its own each time; one expert of four
# without a shared one; a rotation that covers only a part of the rotated values.
_A0 = latent(3, 20, 6, 10, 24, 36, 0.21, 33, base=500.0)
_A1 = latent(2, 12, 10, 28, 40, 18, 0.3, 70, base=10000.0, dims=6)
FID_A = {
    "architecture": "Fidizen", "vocab": 150, "width": 88, "norm": {"eps": 1e-5}, "embedding": {"scale": 7.5}, "canon": {"taps": 3},
    "layers": [
        layer(_A0, moe(5, 2, 24, 40)),
        layer(_A1, None),
        layer(_A0, moe(5, 2, 24, 40), weights_of=0),
        layer(latent(1, 16, 4, 16, 16, 16, 0.25, 0), moe(4, 1, 16)),      # no window: every earlier token
        layer(_A1, None, weights_of=1),
        layer(latent(4, 8, 8, 8, 32, 24, 0.4, 5), dense(72)),             # a window shorter than the taps' reach matters little: 5 tokens
    ],
}

# Sizes the tensor-core kernels and the vector loads accept: keys of 64 + 32 and 32 + 16 values, experts grouped on the tensor
# cores; two taps; all experts of three; a window of exactly one page and one of 100
_B0 = latent(4, 32, 32, 48, 64, 64, 0.125, 64)
FID_B = {
    "architecture": "Fidizen", "vocab": 320, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 16.0}, "canon": {"taps": 2},
    "layers": [
        layer(_B0, dense(384)),
        layer(latent(8, 16, 16, 32, 96, 32, 0.18, 100), moe(6, 2, 64, 128)),
        layer(_B0, dense(384), weights_of=0),
        layer(latent(2, 64, 64, 64, 32, 128, 0.09, 150), moe(3, 3, 128, 64)),
    ],
}

# One layer, one head, one tap (a convolution that sees nothing but the token itself), no embedding scale, a window of one
FID_C = {
    "architecture": "Fidizen", "vocab": 64, "width": 48, "norm": {"eps": 1e-6}, "canon": {"taps": 1},
    "layers": [layer(latent(1, 24, 2, 40, 8, 12, 0.3, 1), dense(40)), layer(latent(2, 4, 12, 6, 20, 10, 0.5, 2), moe(2, 1, 8, 8))],
}


def config(which):
    return copy.deepcopy({"a": FID_A, "b": FID_B, "c": FID_C}[which])
