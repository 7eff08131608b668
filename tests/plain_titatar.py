"""A plain, slow implementation of the Titatar design: float64, one function per mechanism, token lists in,
logits out.  It shares no code with the package; the tests compare the package with it.

Notation: x is the residual stream [tokens, width]; h a sublayer's input; W matrices are [out, in] and applied
as W h; positions count from 0.  Weights come in as a dict name -> float64 array, the configuration as the
nested document of config.json.
"""
from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    """The design's norm: weights are stored around zero."""
    return rms(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def frequencies(rot):
    """Turning rate of every pair, with the long wavelengths stretched if the document asks for it; and the factor
    on cosines and sines."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    s = rot.get("scaling")
    if not s:
        return f, 1.0
    factor, original = float(s["factor"]), float(s["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(float(s["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(s["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v, positions, rot, interleaved):
    """v [tokens, heads, n]: the first rot.dims entries of each head are rotated, the rest pass; no ``rot``, no rotation."""
    dims = int(rot["dims"]) if rot else 0
    if dims == 0:
        return v
    f, mag = frequencies(rot)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]          # [tokens, dims/2]
    c, s = (np.cos(angle) * mag)[:, None, :], (np.sin(angle) * mag)[:, None, :]
    out = v.copy()
    if interleaved:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = v[..., :dims // 2], v[..., dims // 2:dims]
        out[..., :dims // 2] = a * c - b * s
        out[..., dims // 2:dims] = b * c + a * s
    return out


def attend(q, k, v, scale, window, sink):
    """q [T, H, d], k [T, H, d], v [T, H, dv] of one sequence (keys already per query head); ``window`` None = all
    keys up to the row's own; ``sink`` [H]: exp(sink_h) joins the denominator."""
    tokens, heads = q.shape[0], q.shape[1]
    out = np.zeros((tokens, heads, v.shape[2]))
    for i in range(tokens):
        first = 0 if window is None else max(0, i - window + 1)
        for h in range(heads):
            s = (k[first:i + 1, h] @ q[i, h]) * scale
            m = max(s.max(), sink[h])
            e = np.exp(s - m)
            out[i, h] = (e @ v[first:i + 1, h]) / (e.sum() + math.exp(sink[h] - m))
    return out


def windowed_attention(h, positions, w, p, m, eps):
    """The mixer 'attention': grouped heads, norms over the whole q and k projections, half-split rotation of the
    leading entries, a window, one added to the softmax's denominator, a gate per head."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]
    k = rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    q = rotate(q.reshape(T, H, d), positions, m.get("rot"), False)
    k = rotate(k.reshape(T, G, d), positions, m.get("rot"), False)
    per = H // G
    kq = np.repeat(k, per, axis=1)
    vq = np.repeat(v, per, axis=1)
    mask = m.get("mask")
    o = attend(q, kq, vq, m["scale"], int(mask["size"]) if mask else None, np.zeros(H))
    o = o * sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def latent_attention(h, positions, w, p, m, eps):
    """The mixer 'latent_attention': queries through a normed latent, keys and values from a normed latent plus one
    rotated key part for all heads, interleaved rotation, a learned sink per head, a gate per entry."""
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + r)
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = rotate(down[:, None, rank:], positions, m.get("rot"), True)               # [T, 1, r]
    q_rot = rotate(q[:, :, d:], positions, m.get("rot"), True)
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    qq = np.concatenate([q[:, :, :d], q_rot], axis=2)
    kk = np.concatenate([k_plain, np.repeat(k_rot, H, axis=1)], axis=2)
    o = attend(qq, kk, v, m["scale"], None, w[p + "sink"])
    o = o.reshape(T, H * dv) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def gated(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed(h, w, p, f):
    """Experts chosen per token: softmax over all router outputs, the choice by score + correction, the weights the
    scores themselves; the last ``identity`` outputs stand for experts that return their input; a shared expert."""
    r = f["router"]
    real, ident, top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
    z = h @ w[p + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(axis=-1, keepdims=True)
    choice = s + w[p + "correction"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(real + ident), key=lambda e: (-choice[t, e], e))[:top]
        for e in order:
            out[t] += s[t, e] * (gated(h[t:t + 1], w, f"{p}e{e}.")[0] if e < real else h[t])
    if f.get("shared"):
        out += gated(h, w, p + "shared.")
    return out


def layer_runs(cfg):
    """The order in which layers run: (layer, opens a later pass)."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, collect=None):
    """Logits [tokens, vocab] of one sequence fed whole; ``collect`` (a list) receives the stream after each layer run."""
    eps = cfg["norm"]["eps"]
    positions = np.arange(len(tokens))
    x0 = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    x = x0.copy()
    for index, reopen in layer_runs(cfg):
        spec, p = cfg["layers"][index], f"l{index}."
        if reopen:
            x = x + x0
        h = norm_one_plus(x, w[p + "norm1"], eps)
        mixer = windowed_attention if spec["type"] == "attention" else latent_attention
        x = x + norm_one_plus(mixer(h, positions, w, p + "mix.", spec["mixer"], eps), w[p + "norm1b"], eps)
        f = spec.get("mlp")
        if f:
            h = norm_one_plus(x, w[p + "norm2"], eps)
            y = gated(h, w, p + "mlp.") if f["kind"] == "dense" else routed(h, w, p + "mlp.", f)
            x = x + norm_one_plus(y, w[p + "norm2b"], eps)
        if collect is not None:
            collect.append(x.copy())
    return norm_one_plus(x, w["final.norm"], eps) @ w["head"].T
