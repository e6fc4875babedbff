"""Plain, slow restatement of the Vozetar decoder in numpy float64: whole sequences, no cache, no state carried between
calls, one function per mechanism, nothing imported from the package under test (the model-folder reader is the
tests' own).  The GPU tests compare the library with these functions.

Notation: n tokens of one sequence at places 0 .. n-1; matrices are stored [out, in]; `w` maps tensor names (without the
layer's prefix) to arrays."""
from __future__ import annotations

import numpy as np

from plain_llama import read_model  # noqa: F401  (config dict, name -> array)

D64 = np.float64


def unit_rms(x, eps):
    x = np.asarray(x, D64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, scale, eps):
    return unit_rms(x, eps) * np.asarray(scale, D64)


def lin(x, w, b=None):
    y = np.asarray(x, D64) @ np.asarray(w, D64).T
    return y if b is None else y + np.asarray(b, D64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, D64)))


def silu(z):
    z = np.asarray(z, D64)
    return z * sigmoid(z)


# ----------------------------------------------------------------------------- embedding
def embed_tokens(tokens, table, pair_table, pairs):
    """Row of the token plus a row of the pair table chosen by (previous, current); a sequence's first token takes the last row."""
    x = np.asarray(table, D64)[np.asarray(tokens)]
    if pair_table is None:
        return x
    pair_table = np.asarray(pair_table, D64)
    n_rows = int(pairs["buckets"])
    out = x.copy()
    for t, tok in enumerate(tokens):
        row = n_rows if t == 0 else (int(tokens[t - 1]) * int(pairs["mul_prev"]) + int(tok) * int(pairs["mul_cur"])) % n_rows
        out[t] += pair_table[row]
    return out


# ----------------------------------------------------------------------------- pieces of the mixers
def short_convolution(u, taps):
    """Causal convolution over time per channel: u [n, c], taps [c, k]; tap j weighs the token k - 1 - j places back."""
    u = np.asarray(u, D64)
    taps = np.asarray(taps, D64)
    n, k = u.shape[0], taps.shape[1]
    out = np.zeros_like(u)
    for t in range(n):
        for j in range(k):
            src = t - (k - 1) + j
            if src >= 0:
                out[t] += taps[:, j] * u[src]
    return out


def turn(x, dims, base, pairing):
    """Rotary positions on the first `dims` values of every head: x [n, heads, d].  pairing "interleaved": values 2i, 2i + 1
    form a pair; "half": values i, i + dims / 2.  Pair i at place p turns by p * base^(-2i / dims)."""
    x = np.asarray(x, D64)
    out = x.copy()
    p = np.arange(x.shape[0], dtype=D64)[:, None]
    for i in range(dims // 2):
        a, b = (2 * i, 2 * i + 1) if pairing == "interleaved" else (i, i + dims // 2)
        ang = p * float(base) ** (-2.0 * i / dims)
        c, s = np.cos(ang), np.sin(ang)
        out[:, :, a] = x[:, :, a] * c - x[:, :, b] * s
        out[:, :, b] = x[:, :, b] * c + x[:, :, a] * s
    return out


def visible(i, j, window=None, keep_first=0):
    if j > i:
        return False
    return window is None or i - j < window or j < keep_first


def softmax_attention(q, k, v, scale, window=None, keep_first=0, sink=None):
    """q [n, H, d], k [n, G, d], v [n, G, dv]; query head h reads key head h // (H / G); with a sink the denominator holds
    exp(sink_h) once more."""
    q, k, v = (np.asarray(a, D64) for a in (q, k, v))
    n, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((n, H, v.shape[2]), D64)
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            js = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
            s = np.array([q[i, h] @ k[j, g] for j in js]) * scale
            m = s.max() if sink is None else max(s.max(), float(sink[h]))
            e = np.exp(s - m)
            den = e.sum() + (0.0 if sink is None else np.exp(float(sink[h]) - m))
            out[i, h] = (e / den) @ v[js, g]
    return out


def decayed_memory(q, k, v, decay):
    """Per head S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [n, H, d], v [n, H, dv], decay [n, H, d]."""
    q, k, v, decay = (np.asarray(a, D64) for a in (q, k, v, decay))
    n, H, d = q.shape
    out = np.zeros((n, H, v.shape[2]), D64)
    for h in range(H):
        S = np.zeros((d, v.shape[2]), D64)
        for t in range(n):
            S = decay[t, h][:, None] * S + np.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def heads_of(x, heads):
    return np.asarray(x, D64).reshape(x.shape[0], heads, -1)


# ----------------------------------------------------------------------------- the three mixers
def softmax_branch(h, w, m, eps, *, bias, taps_on, qk_norm, pairing, sink, values_are_keys):
    """A softmax attention branch with its options; returns the heads' outputs [n, H, dv] before gate and output product."""
    H, G = m["heads"], m["kv_heads"]
    q = lin(h, w["q"], w.get("q.b") if bias else None)
    k = lin(h, w["k"], w.get("k.b") if bias else None)
    v = None if values_are_keys else lin(h, w["v"], w.get("v.b") if bias else None)
    if taps_on:
        q = short_convolution(q, w["q.conv"])
        k = short_convolution(k, w["k.conv"])
        if v is not None:
            v = short_convolution(v, w["v.conv"])
    if values_are_keys:
        v = k
    if qk_norm:
        q = rms_norm(q, w["q.norm"], eps)
        k = rms_norm(k, w["k.norm"], eps)
    qh = turn(heads_of(q, H), m["rot"]["dims"], m["rot"]["base"], pairing)
    kh = turn(heads_of(k, G), m["rot"]["dims"], m["rot"]["base"], pairing)
    mask = m.get("mask")
    return softmax_attention(qh, kh, heads_of(v, G), m["scale"], mask["size"] if mask else None, mask["keep_first"] if mask else 0,
                             w["sink"] if sink else None)


def mixer_attention(h, w, m, eps):
    o = softmax_branch(h, w, m, eps, bias=True, taps_on=True, qk_norm=False, pairing="half", sink=True, values_are_keys=False)
    o = o.reshape(o.shape[0], -1) * sigmoid(lin(h, w["g"]))
    return lin(o, w["o"], w["o.b"])


def retention_branch(h, w, m, eps):
    H, d = m["heads"], m["dim"]
    q = turn(heads_of(lin(h, w["q"]), H), m["rot"]["dims"], m["rot"]["base"], "half")
    k = turn(heads_of(lin(h, w["k"]), H), m["rot"]["dims"], m["rot"]["base"], "half") * d ** -0.5
    v = heads_of(lin(h, w["v"]), H)
    decay = np.broadcast_to(np.asarray(m["decay"], D64)[None, :, None], q.shape)
    o = unit_rms(decayed_memory(q, k, v, decay), eps)
    return lin(o.reshape(o.shape[0], -1) * silu(lin(h, w["g"])), w["o"])


def gated_memory_branch(h, w, m, eps):
    H, d = m["heads"], m["dim"]
    q = heads_of(lin(h, w["q"]), H) * d ** -0.5
    k = heads_of(lin(h, w["k"]), H)
    v = heads_of(lin(h, w["v"]), H)
    z = lin(lin(h, w["a1"]), w["a2"], w["a2.b"])
    decay = heads_of(sigmoid(z) ** (1.0 / m["tau"]), H)
    o = rms_norm(decayed_memory(q, k, v, decay), w["norm"], eps)
    return lin(o.reshape(o.shape[0], -1) * silu(lin(h, w["g"])), w["o"])


def sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def mixer_parallel(h, w, m, eps):
    wl, wr = sub(w, "left."), sub(w, "right.")
    o = softmax_branch(h, wl, m["left"], eps, bias=True, taps_on=False, qk_norm=False, pairing="interleaved", sink=True,
                       values_are_keys=False)
    left = lin(o.reshape(o.shape[0], -1), wl["o"])
    return m["left_scale"] * left + m["right_scale"] * retention_branch(h, wr, m["right"], eps)


def mixer_parallel_2(h, w, m, eps):
    wl, wr = sub(w, "left."), sub(w, "right.")
    o = softmax_branch(h, wl, m["left"], eps, bias=False, taps_on=True, qk_norm=True, pairing="interleaved", sink=False,
                       values_are_keys=True)
    o = o * sigmoid(lin(h, wl["g"]))[:, :, None]
    left = lin(o.reshape(o.shape[0], -1), wl["o"])
    right = gated_memory_branch(h, wr, m["right"], eps)
    return 0.5 * (rms_norm(left, wl["out"], eps) + rms_norm(right, wr["out"], eps))


MIXERS = {"attention": mixer_attention, "parallel": mixer_parallel, "parallel_2": mixer_parallel_2}


# ----------------------------------------------------------------------------- feed-forward
def gated_unit(h, w):
    return lin(silu(lin(h, w["gate"])) * lin(h, w["up"]), w["down"])


def choose_experts(scores, top, groups=None):
    """Indices of the `top` largest scores (ties to the lower index); with groups only experts of the best `keep` groups,
    a group's score being the sum of its two largest scores."""
    s = np.asarray(scores, D64).copy()
    if groups and groups["count"] > 1:
        size = len(s) // groups["count"]
        gs = [np.sort(s[g * size:(g + 1) * size])[-2:].sum() for g in range(groups["count"])]
        order = sorted(range(groups["count"]), key=lambda g: (-gs[g], g))
        for g in order[groups["keep"]:]:
            s[g * size:(g + 1) * size] = -np.inf
    return sorted(range(len(s)), key=lambda e: (-s[e], e))[:top]


def routed_unit(h, w, mlp):
    h = np.asarray(h, D64)
    r = mlp["router"]
    scores = sigmoid(lin(h, w["router"]))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in choose_experts(scores[t], r["top"], r.get("groups")):
            out[t] += scores[t, e] * gated_unit(h[t:t + 1], sub(w, "e%d." % e))[0]
    if mlp.get("shared"):
        out += gated_unit(h, sub(w, "shared."))
    return out


def feed_forward(h, w, mlp):
    return gated_unit(h, w) if mlp["kind"] == "dense" else routed_unit(h, w, mlp)


# ----------------------------------------------------------------------------- layers with several residual streams
def sublayer_on_streams(xs, w_in, w_out, w_mix, norm_w, eps, fn):
    """xs [S, n, width].  The sublayer reads the norm of sum_s in[s] x_s; stream t becomes sum_s mix[s, t] x_s + out[t] y."""
    xs = np.asarray(xs, D64)
    u = np.tensordot(np.asarray(w_in, D64), xs, axes=(0, 0))
    y = fn(rms_norm(u, norm_w, eps))
    return np.tensordot(np.asarray(w_mix, D64).T, xs, axes=(1, 0)) + np.asarray(w_out, D64)[:, None, None] * y[None]


def forward(config, weights, tokens, return_layers=False):
    """Logits [n, vocab] of one sequence (and, if asked, the sum of the streams after every layer)."""
    eps = config["norm"]["eps"]
    big = (config.get("embedding") or {}).get("bigram")
    x = embed_tokens(tokens, weights["embed"], weights.get("bigram") if big else None, big)
    S = int(config.get("streams", 1))
    xs = np.repeat(x[None], S, axis=0)
    after = []
    for i, layer in enumerate(config["layers"]):
        w = sub(weights, "l%d." % i)
        mix = MIXERS[layer["type"]]
        if S > 1 or "hc1.in" in w:
            xs = sublayer_on_streams(xs, w["hc1.in"], w["hc1.out"], w["hc1.mix"], w["norm1"], eps,
                                     lambda a: mix(a, sub(w, "mix."), layer["mixer"], eps))
            if layer.get("mlp"):
                xs = sublayer_on_streams(xs, w["hc2.in"], w["hc2.out"], w["hc2.mix"], w["norm2"], eps,
                                         lambda a: feed_forward(a, sub(w, "mlp."), layer["mlp"]))
        else:
            xs = xs + mix(rms_norm(xs[0], w["norm1"], eps), sub(w, "mix."), layer["mixer"], eps)[None]
            if layer.get("mlp"):
                xs = xs + feed_forward(rms_norm(xs[0], w["norm2"], eps), sub(w, "mlp."), layer["mlp"])[None]
        after.append(xs.sum(axis=0))
    logits = lin(rms_norm(xs.sum(axis=0), weights["final.norm"], eps), weights["head"])
    return (logits, np.stack(after)) if return_layers else logits
