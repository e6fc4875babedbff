"""Plain, slow restatement of the Fidizen decoder in numpy float64: whole sequences, no cache, no state carried between
calls, one function per mechanism, nothing imported from the package under test (the model-folder reader is the
tests' own).  The GPU tests compare the library with these functions.

Notation: n tokens of one sequence at places 0 .. n-1; matrices are stored [out, in]."""
from __future__ import annotations

import numpy as np

from plain_llama import read_model  # noqa: F401  (config dict, name -> array)

D64 = np.float64


def unit_rms(x, eps):
    x = np.asarray(x, D64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, scale, eps):
    return unit_rms(x, eps) * np.asarray(scale, D64)


def lin(x, w):
    return np.asarray(x, D64) @ np.asarray(w, D64).T


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, D64)))


def silu(z):
    z = np.asarray(z, D64)
    return z * sigmoid(z)


# ----------------------------------------------------------------------------- what a sublayer reads
def through_convolution(h, taps):
    """h [n, width] plus, on every channel, the weighted sum of the token itself and the taps - 1 tokens before it:
    tap j weighs the token (taps - 1 - j) places back; nothing lies before place 0."""
    h = np.asarray(h, D64)
    taps = np.asarray(taps, D64)
    n, k = h.shape[0], taps.shape[1]
    out = h.copy()
    for t in range(n):
        for j in range(k):
            src = t - (k - 1 - j)
            if src >= 0:
                out[t] += taps[:, j] * h[src]
    return out


# ----------------------------------------------------------------------------- the mixer
def turn_pairs(x, places, dims, base):
    """Rotary positions on the first `dims` values of the last axis: values 2i and 2i + 1 form a pair that turns by the
    angle place * base^(-2i / dims); the rest passes.  x [n, ..., d], places [n]."""
    x = np.asarray(x, D64)
    out = x.copy()
    places = np.asarray(places, D64).reshape((-1,) + (1,) * (x.ndim - 2))
    for i in range(dims // 2):
        ang = places * base ** (-2.0 * i / dims)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * np.cos(ang) - v * np.sin(ang)
        out[..., 2 * i + 1] = v * np.cos(ang) + u * np.sin(ang)
    return out


def latent_attention(x, w, p, m, eps, return_weights=False):
    """x [n, width] -> [n, width].  m: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {base, dims}, mask {size} (optional)."""
    x = np.asarray(x, D64)
    n, H, d, r, dv, rank = x.shape[0], m["heads"], m["dim"], m.get("rot_dim", 0), m["vdim"], m["kv_rank"]
    places = np.arange(n)
    q = lin(rms_norm(lin(x, w[p + "dq"]), w[p + "dq.norm"], eps), w[p + "uq"]).reshape(n, H, d + r)
    down = lin(x, w[p + "dkv"])
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k = lin(c, w[p + "uk"]).reshape(n, H, d)
    v = lin(c, w[p + "uv"]).reshape(n, H, dv)
    score = np.einsum("ihd,jhd->hij", q[:, :, :d], k)
    if r:
        q_rot = turn_pairs(q[:, :, d:], places, m["rot"]["dims"], m["rot"]["base"])
        k_rot = turn_pairs(down[:, rank:], places, m["rot"]["dims"], m["rot"]["base"])      # one part for all heads
        score = score + np.einsum("ihd,jd->hij", q_rot, k_rot)
    score = score * m["scale"]
    i, j = places[:, None], places[None, :]
    seen = j <= i
    if m.get("mask") and m["mask"].get("size"):
        seen &= (i - j) < m["mask"]["size"]
    sink = np.asarray(w[p + "sink"], D64)
    top = np.maximum(np.where(seen[None], score, -np.inf).max(axis=-1), sink[:, None])
    e = np.where(seen[None], np.exp(score - top[..., None]), 0.0)
    weights = e / (e.sum(axis=-1) + np.exp(sink[:, None] - top))[..., None]      # the sink takes its share and gives nothing
    heads = np.einsum("hij,jhd->ihd", weights, v).reshape(n, H * dv)
    y = lin(heads * sigmoid(lin(x, w[p + "g"])), w[p + "o"])
    return (y, weights) if return_weights else y


# ----------------------------------------------------------------------------- feed-forwards
def polynorm(z, coef, eps):
    z = np.asarray(z, D64)
    a, b, c, e = (float(t) for t in np.asarray(coef, D64))
    return a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e


def dense(x, w, p, eps):
    return lin(polynorm(lin(x, w[p + "up"]), w[p + "act"], eps), w[p + "down"])


def gated_expert(x, w, p):
    return lin(silu(lin(x, w[p + "gate"])) * lin(x, w[p + "up"]), w[p + "down"])


def route(x, w, p, top):
    """(chosen [n, top], weights [n, top]): the experts with the largest sigmoid scores (the lower index wins a tie), their scores as
    weights."""
    s = sigmoid(lin(np.asarray(x, np.float32), np.asarray(w[p + "router"], np.float32)))
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def routed_experts(x, w, p, mlp):
    x = np.asarray(x, D64)
    chosen, weight = route(x, w, p, mlp["router"]["top"])
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        for e, s in zip(chosen[t], weight[t]):
            y[t] += gated_expert(s * x[t][None], w, f"{p}e{int(e)}.")[0]      # the weight goes INTO the expert
    if mlp.get("shared"):
        y += gated_expert(x, w, p + "shared.")
    return y


# ----------------------------------------------------------------------------- the model
def layer(x, w, p, spec, eps, taps):
    """x + norm1(mixer(in(x))), then the same with the feed-forward, if the layer has one."""
    read = through_convolution(x, w[p + "canon1"]) if taps else x
    x = x + rms_norm(latent_attention(read, w, p + "mix.", spec["mixer"], eps), w[p + "norm1"], eps)
    mlp = spec.get("mlp")
    if mlp:
        read = through_convolution(x, w[p + "canon2"]) if taps else x
        y = dense(read, w, p + "mlp.", eps) if mlp["kind"] == "dense" else routed_experts(read, w, p + "mlp.", mlp)
        x = x + rms_norm(y, w[p + "norm2"], eps)
    return x


def forward_logits(cfg, w, tokens, streams=None):
    eps = cfg["norm"]["eps"]
    taps = (cfg.get("canon") or {}).get("taps", 0)
    x = np.asarray(w["embed"], D64)[list(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    for i, spec in enumerate(cfg["layers"]):
        src = i
        while cfg["layers"][src].get("weights_of") is not None:
            src = cfg["layers"][src]["weights_of"]
        x = layer(x, w, f"l{src}.", cfg["layers"][src], eps, taps)
        if streams is not None:
            streams.append(x.copy())
    return lin(rms_norm(x, w["final.norm"], eps), w["head"])


def generate_greedy(cfg, w, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(np.argmax(forward_logits(cfg, w, seq)[-1])))
    return seq[len(prompt):]
