"""Plain, slow restatement of the Mokatar decoder, used only as a test oracle.

Whole sequences, no cache, one function per mechanism, float64 throughout, no code shared with the product
package.  Notation: h is a sublayer's input [T, width]; p the positions 0..T-1; a weight matrix is [out, in] and
acts as h @ W.T; cfg is the config.json object, W a dict name -> array.

  embedding      x0 = E[tok] * scale + B[(prev * m_prev + tok * m_cur) mod buckets], a sequence's first token reads
                 row `buckets` of B
  layer          x += mixer(n1(x)) + ff(n2(x)), both sublayers on the same x;  n(x) = x / rms(x) * (1 + w)
  loop           layers start .. stop - 1 run `times` times with the same weights; pass t begins with
                 x += x0 (t > 0), then x += step[t]
  attention      q, k, v = Wq h, Wk h, Wv h;  per head q, k <- rms over the head * g (one g for all heads);  the
                 first n dimensions of every head turned in pairs (2i, 2i + 1) by p * f_i, f from the YaRN ramp, cos
                 and sin times 0.1 ln(factor) + 1;  position p sees t <= p with p - t < size or t < keep_first;
                 a_t = exp(s_t) / (sum exp(s) + exp(sink_head));  Wo
  attention_2    biases on q, k, v;  q and k each rms-normed over the whole projection (all heads at once) with a gain
                 per column;  pairs (i, i + n/2), f_i / factor;  causal;  a_t = exp(s_t) / (1 + sum exp(s));  Wo
  gla            q = Wq h / sqrt(d), k = Wk h, v = Wv h;  alpha = sigmoid(Wa2 (Wa1 h) + b)^(1/tau) per key channel;
                 S <- diag(alpha) S + k v^T;  o = S^T q;  per head o / rms(o) * g;  times silu(Wg h);  Wo
  feed-forward   Wd (silu(Wg h) * (Wu h)), or the `top` experts by router logit Wr h + b, weighted by the softmax over
                 the chosen logits only
  output         logits = head (final norm(x)) * logit_scale
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np

F64 = np.float64


def linear(x, w, b=None):
    y = np.asarray(x, F64) @ np.asarray(w, F64).T
    return y if b is None else y + np.asarray(b, F64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, F64)))


def silu(z):
    z = np.asarray(z, F64)
    return z * sigmoid(z)


def rms_norm(x, gain, eps, one_plus=False):
    x = np.asarray(x, F64)
    g = np.asarray(gain, F64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + F64(eps)) * (1.0 + g if one_plus else g)


# ---------------------------------------------------------------------------------------------- embedding
def embed(cfg, W, tokens):
    e = cfg.get("embedding") or {}
    big, scale = e.get("bigram"), e.get("scale", 1.0)
    table = np.asarray(W["embed"], F64)
    out = np.zeros((len(tokens), table.shape[1]), F64)
    for i, tok in enumerate(tokens):
        out[i] = table[tok] * scale
        if big is not None:                   # a model without a pair table adds nothing
            row = big["buckets"] if i == 0 else (tokens[i - 1] * big["mul_prev"] + tok * big["mul_cur"]) % big["buckets"]
            out[i] += np.asarray(W["bigram"][row], F64)
    return out


# ---------------------------------------------------------------------------------------------- rotation
def frequencies(rot):
    """(f [dims / 2], magnitude of cos and sin) of a mixer's `rot` object; none at all: nothing is turned."""
    if not rot or not rot.get("dims"):
        return np.zeros(0, F64), 1.0
    n, base = rot["dims"], float(rot["base"])
    f = np.array([base ** (-2.0 * i / n) for i in range(n // 2)], F64)
    sc = rot.get("scaling") or {}
    if "original" in sc:                      # the ramp between scaled and unscaled frequencies
        factor = float(sc["factor"])

        def dim_of(turns):
            return n * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(dim_of(sc["fast"])), 0)
        hi = min(math.ceil(dim_of(sc["slow"])), n - 1)
        ramp = np.clip((np.arange(n // 2, dtype=F64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0
    if "factor" in sc:
        return f / float(sc["factor"]), 1.0
    return f, 1.0


def rotate(x, positions, f, mag, neighbours):
    """x [T, heads, d]: the first 2 len(f) dimensions of every head are turned; neighbours: pairs (2i, 2i + 1),
    else (i, i + len(f))."""
    x = np.array(x, F64)
    n = len(f)
    ang = np.asarray(positions, F64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    if neighbours:
        u, v = x[..., 0:2 * n:2].copy(), x[..., 1:2 * n:2].copy()
        x[..., 0:2 * n:2], x[..., 1:2 * n:2] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., :n].copy(), x[..., n:2 * n].copy()
        x[..., :n], x[..., n:2 * n] = u * c - v * s, v * c + u * s
    return x


# ---------------------------------------------------------------------------------------------- attention
def masked_softmax_attention(q, k, v, scale, sink, size, keep_first):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; sink [H] (the score of a term without key or value in every
    denominator); size 0: every earlier key, else the last `size` and the first `keep_first`."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        i, j = np.arange(T)[:, None], np.arange(T)[None, :]
        seen = j <= i
        if size:
            seen &= (i - j < size) | (j < keep_first)
        s = np.where(seen, s, -np.inf)
        m = np.maximum(s.max(axis=1, keepdims=True), sink[h])
        e = np.exp(s - m)
        out[:, h] = (e / (e.sum(axis=1, keepdims=True) + np.exp(sink[h] - m))) @ v[:, g]
    return out


def attention(m, W, pre, h, eps, positions=None):
    T = h.shape[0]
    p = np.arange(T) if positions is None else positions
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, W[pre + "q"]).reshape(T, H, d)
    k = linear(h, W[pre + "k"]).reshape(T, G, d)
    v = linear(h, W[pre + "v"]).reshape(T, G, dv)
    q, k = rms_norm(q, W[pre + "q.norm"], eps), rms_norm(k, W[pre + "k.norm"], eps)
    f, mag = frequencies(m.get("rot"))
    q, k = rotate(q, p, f, mag, True), rotate(k, p, f, mag, True)
    mask = m.get("mask") or {}
    o = masked_softmax_attention(q, k, v, m["scale"], np.asarray(W[pre + "sink"], F64), mask.get("size", 0),
                                 mask.get("keep_first", 0))
    return linear(o.reshape(T, H * dv), W[pre + "o"])


def attention_2(m, W, pre, h, eps, positions=None):
    T = h.shape[0]
    p = np.arange(T) if positions is None else positions
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(linear(h, W[pre + "q"], W[pre + "q.b"]), W[pre + "q.norm"], eps).reshape(T, H, d)
    k = rms_norm(linear(h, W[pre + "k"], W[pre + "k.b"]), W[pre + "k.norm"], eps).reshape(T, G, d)
    v = linear(h, W[pre + "v"], W[pre + "v.b"]).reshape(T, G, dv)
    f, mag = frequencies(m.get("rot"))
    q, k = rotate(q, p, f, mag, False), rotate(k, p, f, mag, False)
    o = masked_softmax_attention(q, k, v, m["scale"], np.zeros(H, F64), 0, 0)
    return linear(o.reshape(T, H * dv), W[pre + "o"])


# ---------------------------------------------------------------------------------------------- gated linear attention
def gla_decay(m, W, pre, h):
    z = linear(linear(h, W[pre + "a1"]), W[pre + "a2"], W[pre + "a2.b"])
    return sigmoid(z) ** (1.0 / m["tau"])


def gla_recurrence(q, k, v, alpha, state=None):
    """q, k, alpha [T, H, d], v [T, H, dv]; token by token, as the rule is stated.  Returns (o [T, H, dv], S)."""
    T, H, d = q.shape
    S = np.zeros((H, d, v.shape[2]), F64) if state is None else np.array(state, F64)
    o = np.zeros((T, H, v.shape[2]), F64)
    for t in range(T):
        for j in range(H):
            S[j] = alpha[t, j][:, None] * S[j] + np.outer(k[t, j], v[t, j])
            o[t, j] = S[j].T @ q[t, j]
    return o, S


def gla(m, W, pre, h, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = linear(h, W[pre + "q"]).reshape(T, H, d) * d ** -0.5
    k = linear(h, W[pre + "k"]).reshape(T, H, d)
    v = linear(h, W[pre + "v"]).reshape(T, H, dv)
    o, _ = gla_recurrence(q, k, v, gla_decay(m, W, pre, h).reshape(T, H, d))
    o = rms_norm(o, W[pre + "norm"], eps).reshape(T, H * dv)
    return linear(o * silu(linear(h, W[pre + "g"])), W[pre + "o"])


# ---------------------------------------------------------------------------------------------- feed-forward
def gated_ff(W, pre, h):
    return linear(silu(linear(h, W[pre + "gate"])) * linear(h, W[pre + "up"]), W[pre + "down"])


def route(f, W, pre, h, margins=None):
    """(chosen [T, top], weights [T, top]): the largest logits, and the softmax over those alone.  margins (a list):
    every token's gap between the last chosen logit and the best one left out is appended."""
    z = linear(h, W[pre + "router"], W[pre + "router.b"])
    top = f["router"]["top"]
    chosen = np.argsort(-z, axis=1, kind="stable")[:, :top]
    if margins is not None and top < z.shape[1]:
        ordered = -np.sort(-z, axis=1)
        margins.extend((ordered[:, top - 1] - ordered[:, top]).tolist())
    zc = np.take_along_axis(z, chosen, axis=1)
    e = np.exp(zc - zc.max(axis=1, keepdims=True))
    return chosen, e / e.sum(axis=1, keepdims=True)


def routed_ff(f, W, pre, h, margins=None):
    chosen, weights = route(f, W, pre, h, margins)
    out = np.zeros((h.shape[0], np.asarray(W[pre + "e0.down"]).shape[0]), F64)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * gated_ff(W, f"{pre}e{e}.", h[t:t + 1])[0]
    return out


def feed_forward(f, W, pre, h, margins=None):
    return gated_ff(W, pre, h) if f["kind"] == "dense" else routed_ff(f, W, pre, h, margins)


# ---------------------------------------------------------------------------------------------- the model
MIXERS = {"attention": attention, "attention_2": attention_2, "gla": gla}


def layer(cfg, W, i, x, margins=None):
    entry = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    pre = f"l{i}."
    y = MIXERS[entry["type"]](entry["mixer"], W, pre + "mix.", rms_norm(x, W[pre + "norm1"], eps, True), eps)
    if entry.get("mlp") is not None:
        y = y + feed_forward(entry["mlp"], W, pre + "mlp.", rms_norm(x, W[pre + "norm2"], eps, True), margins)
    return x + y


def runs(cfg):
    """(layer, pass or None if the layer is outside the loop, first of its pass) in running order."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, None, False) for i in range(n)]
    out = [(i, None, False) for i in range(lp["start"])]
    for t in range(lp["times"]):
        out += [(i, t, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return out + [(i, None, False) for i in range(lp["stop"], n)]


def forward(cfg, W, tokens, streams: Optional[List[np.ndarray]] = None, margins: Optional[list] = None):
    """Logits [T, vocab] of one sequence from its first token; streams (a list): the residual stream after every
    layer run is appended; margins (a list): every routing decision's gap between chosen and not chosen."""
    x0 = embed(cfg, W, tokens)
    x = x0.copy()
    for i, t, first in runs(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + np.asarray(W["loop.step"], F64)[t]
        x = layer(cfg, W, i, x, margins)
        if streams is not None:
            streams.append(x.copy())
    xn = rms_norm(x, W["final.norm"], cfg["norm"]["eps"], True)
    return linear(xn, W["head"]) * cfg["logit_scale"]


def greedy(cfg, W, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(np.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]
