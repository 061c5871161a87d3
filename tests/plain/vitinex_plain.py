"""Plain, slow restatement of the Vitinex decoder, used only as a test oracle.

Whole sequences, no cache, one function per mechanism, float64 throughout, no code shared with the product
package.  Notation: h is a sublayer's input [T, width]; p the positions 0..T-1; a weight matrix is [out, in] and
acts as h @ W.T.

  layer               x += m LN1b(mixer(LN1(x)));  x += m LN2b(ff(LN2(x))):  a norm on either side of every sublayer
  LN                  (y - mean(y)) / sqrt(var(y) + eps) * w   (no bias; var = mean of the squared deviations)
  loop                layers start .. stop - 1 run `times` times with the same weights; at the head of pass t
                      x = W_loop [x ; x0] + step[t], x0 the embedded tokens
  latent attention    cq = rms(Wdq h) gq;  q = Wuq cq, per head [d plain | r rotated];  Wdkv h = [c' | kr];
                      c = rms(c') gc;  k_j = [Wuk_j c | kr],  v_j = Wuv_j c;  kr and the rotated part of q turned in
                      pairs (2i, 2i + 1) by p * base^(-2i/n);  causal softmax of q . k * scale;  head j's output
                      times sigmoid(Wg h)_j;  Wo
  state-space mixer   W h = [z | x | B | C | dt];  (x, B, C) <- silu(causal_conv + bias);  dt <- softplus(dt + bias);
                      per head (group floor(head / (heads / groups))):  S = exp(-exp(A_log) dt) S + dt B x^T;
                      y = S^T C + D x;  y <- y silu(z);  rms in `norm_groups` equal parts, times w;  Wo
  dense feed-forward  Wd (gelu_tanh(Wg h + bg) * (Wu h + bu)) + bd
  routed experts      z = Wr h;  s = softmax(z);  the `top` largest s are chosen and weigh their experts as they are;
                      expert: Wd relu(Wu h)^2;  + sigmoid(wsg . h) * the shared expert
"""
from __future__ import annotations

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


def softplus(z):
    z = np.asarray(z, F64)
    return np.where(z > 30, z, np.log1p(np.exp(np.minimum(z, 30))))


def gelu_tanh(z):
    z = np.asarray(z, F64)
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, gain, eps):
    x = np.asarray(x, F64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + F64(eps)) * np.asarray(gain, F64)


def layer_norm(x, w, eps):
    x = np.asarray(x, F64)
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + F64(eps)) * np.asarray(w, F64)


def rotate_pairs(x, pos, base, n):
    """x [T, heads, m], m >= n: the pairs (2i, 2i + 1), i < n/2, of every head turned by p * base^(-2i/n)."""
    x = np.array(x, F64)
    i = np.arange(n // 2, dtype=F64)
    f = F64(base) ** (-2.0 * i / F64(n))
    a = np.asarray(pos, F64)[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., 0:n:2].copy(), x[..., 1:n:2].copy()
    x[..., 0:n:2] = u * c - v * s
    x[..., 1:n:2] = v * c + u * s
    return x


def latent_attention(h, w: Dict[str, np.ndarray], m: dict, eps: float):
    """m: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot{base, dims}.  w: dq, dq.norm, uq, dkv, dkv.norm, uk,
    uv, g, o."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    cq = rms_norm(linear(h, w["dq"]), w["dq.norm"], eps)
    q = linear(cq, w["uq"]).reshape(T, H, d + r)
    low = linear(h, w["dkv"])
    c = rms_norm(low[:, :rank], w["dkv.norm"], eps)
    kr = low[:, rank:].reshape(T, 1, r)
    n = m["rot"]["dims"]
    q_rot = rotate_pairs(q[:, :, d:], pos, m["rot"]["base"], n)
    kr = rotate_pairs(kr, pos, m["rot"]["base"], n)
    k_plain = linear(c, w["uk"]).reshape(T, H, d)
    v = linear(c, w["uv"]).reshape(T, H, dv)
    gate = sigmoid(linear(h, w["g"]))                       # [T, H]
    out = np.zeros((T, H, dv), F64)
    causal = pos[None, :] <= pos[:, None]
    for j in range(H):
        s = (q[:, j, :d] @ k_plain[:, j].T + q_rot[:, j] @ kr[:, 0].T) * F64(m["scale"])
        s = np.where(causal, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        a = np.exp(s)
        a = a / a.sum(axis=-1, keepdims=True)
        out[:, j] = (a @ v[:, j]) * gate[:, j:j + 1]
    return linear(out.reshape(T, H * dv), w["o"])


def causal_conv(x, taps, bias):
    """x [T, C], taps [C, n] (the last column is the current token's), zeros before the start."""
    x, taps = np.asarray(x, F64), np.asarray(taps, F64)
    T, n = x.shape[0], taps.shape[1]
    y = np.tile(np.asarray(bias, F64), (T, 1))
    for t in range(T):
        for i in range(n):                                   # the input i tokens back meets column n - 1 - i
            if t - i >= 0:
                y[t] += taps[:, n - 1 - i] * x[t - i]
    return y


def ssm_scan(x, B, C, dt, a_log, D, heads, groups):
    """x [T, heads, P], B and C [T, groups, N], dt [T, heads] (after softplus): y [T, heads, P], token by token."""
    T, _, P = x.shape
    N = B.shape[2]
    per = heads // groups
    y = np.zeros((T, heads, P), F64)
    for j in range(heads):
        g = j // per
        S = np.zeros((N, P), F64)
        A = -np.exp(F64(a_log[j]))
        for t in range(T):
            S = np.exp(A * dt[t, j]) * S + dt[t, j] * np.outer(B[t, g], x[t, j])
            y[t, j] = S.T @ C[t, g] + F64(D[j]) * x[t, j]
    return y


def state_space_mixer(h, w: Dict[str, np.ndarray], m: dict, eps: float):
    """m: heads, vdim, state, groups, conv, norm_groups.  w: in, conv, conv.b, dt_bias, A_log, D, norm, o."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    row = linear(h, w["in"])
    z, xbc, dt = row[:, :inner], row[:, inner:2 * inner + 2 * G * N], row[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + np.asarray(w["dt_bias"], F64))
    y = ssm_scan(x, B, C, dt, np.asarray(w["A_log"], F64), np.asarray(w["D"], F64), H, G).reshape(T, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = y.reshape(T, parts, inner // parts)
    y = y / np.sqrt(np.mean(y * y, axis=-1, keepdims=True) + F64(eps))
    y = y.reshape(T, inner) * np.asarray(w["norm"], F64)
    return linear(y, w["o"])


def dense_feed_forward(h, w):
    return linear(gelu_tanh(linear(h, w["gate"], w["gate.b"])) * linear(h, w["up"], w["up.b"]), w["down"], w["down.b"])


def squared_relu_expert(h, up, down):
    a = np.maximum(linear(h, up), 0.0)
    return linear(a * a, down)


def route_softmax(h, router, top, margins: Optional[list] = None):
    """(chosen [T, top], their scores [T, top]): the largest softmax scores, lower index first among equals.
    margins (a list) receives, per token, the gap between the last chosen logit and the best one left out."""
    z = linear(h, router)
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    full = np.argsort(-s, axis=-1, kind="stable")
    order = full[:, :top]
    if margins is not None and top < z.shape[-1]:
        rows = np.arange(z.shape[0])
        margins.extend((z[rows, full[:, top - 1]] - z[rows, full[:, top]]).tolist())
    return order, np.take_along_axis(s, order, axis=-1)


def routed_experts(h, w: Dict[str, np.ndarray], f: dict, margins: Optional[list] = None):
    T = h.shape[0]
    E, top = f["router"]["experts"], f["router"]["top"]
    chosen, score = route_softmax(h, w["router"], top, margins)
    out = np.zeros((T, np.asarray(w["e0.down"]).shape[0]), F64)
    for t in range(T):
        for k in range(top):
            e = int(chosen[t, k])
            out[t] += score[t, k] * squared_relu_expert(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if f.get("shared"):
        gate = sigmoid(linear(h, w["shared.sg"]))            # [T, 1]
        out += gate * squared_relu_expert(h, w["shared.up"], w["shared.down"])
    assert E == sum(1 for k in w if k.endswith(".up") and k.startswith("e"))
    return out


def sub(weights: Dict[str, np.ndarray], prefix: str) -> Dict[str, np.ndarray]:
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def layer_forward(x, weights, cfg: dict, i: int, margins: Optional[list] = None):
    L, eps, m = cfg["layers"][i], cfg["norm"]["eps"], F64(cfg["residual_mult"])
    p = f"l{i}."
    h = layer_norm(x, weights[p + "norm1"], eps)
    if L["type"] == "latent_attention":
        y = latent_attention(h, sub(weights, p + "mix."), L["mixer"], eps)
    else:
        y = state_space_mixer(h, sub(weights, p + "mix."), L["mixer"], eps)
    x = x + m * layer_norm(y, weights[p + "norm1b"], eps)
    if L.get("mlp") is not None:
        h = layer_norm(x, weights[p + "norm2"], eps)
        f = L["mlp"]
        y = dense_feed_forward(h, sub(weights, p + "mlp.")) if f["kind"] == "dense" else routed_experts(h, sub(weights, p + "mlp."), f, margins)
        x = x + m * layer_norm(y, weights[p + "norm2b"], eps)
    return x


def layer_runs(cfg: dict) -> List[tuple]:
    """(layer, pass or None, first of its pass) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    runs = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None, False) for i in range(loop["stop"], n)]


def forward(tokens, weights: Dict[str, np.ndarray], cfg: dict, streams: Optional[list] = None,
            margins: Optional[list] = None):
    """Logits [T, vocab] of one whole sequence; streams (a list) receives the residual stream after every layer run,
    margins the routers' gaps between the last expert chosen and the first left out (in logits)."""
    x0 = np.asarray(weights["embed"], F64)[np.asarray(tokens)]
    x = x0.copy()
    for i, t, first in layer_runs(cfg):
        if first:
            x = linear(np.concatenate([x, x0], axis=-1), weights["loop.in"]) + np.asarray(weights["loop.step"], F64)[t]
        x = layer_forward(x, weights, cfg, i, margins)
        if streams is not None:
            streams.append(x.copy())
    return linear(layer_norm(x, weights["final.norm"], cfg["norm"]["eps"]), weights["embed"])
