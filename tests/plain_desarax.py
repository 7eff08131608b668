"""A plain, slow implementation of the Desarax design in float64, one function per mechanism.

It shares no code with the package: tensors come in as a dict of name -> torch tensor, the configuration as the
plain document, and every function walks tokens and heads in Python loops where that is the clearest form.
A whole sequence is computed at once (no cache, no portions); the package must give the same logits however the
sequence is cut.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    # log(1 + exp(z)) without overflow
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, weight, groups, eps):
    """RMS norm in ``groups`` equal consecutive parts of the last axis, then the weight over the whole."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    return rms(parts, eps).reshape(shape) * weight


def causal_conv(u, weight, bias):
    """u [T, channels]; weight [channels, taps] whose last column multiplies the current token; zeros before the start."""
    T, channels = u.shape
    taps = weight.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        acc = bias.clone()
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                acc = acc + weight[:, j] * u[s]
        out[t] = acc
    return out


def recurrence(x, B, C, dt, a_log, skip, begin=None):
    """x [T, heads, P], B and C [T, G, N], dt [T, heads] (after the softplus): per head S <- exp(-exp(a_log) dt) S + dt B x^T,
    y = S^T C + skip x, from the states ``begin`` [heads, N, P] (zeros without).  Returns (y [T, heads, P], the last states)."""
    T, heads, P = x.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros(T, heads, P, dtype=F)
    last = torch.zeros(heads, N, P, dtype=F)
    for head in range(heads):
        g = head // (heads // G)
        S = torch.zeros(N, P, dtype=F) if begin is None else begin[head].clone()
        rate = torch.exp(a_log[head])
        for t in range(T):
            S = torch.exp(-rate * dt[t, head]) * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + skip[head] * x[t, head]
        last[head] = S
    return y, last


def mamba2(h, w, m, eps):
    """The state-space mixer over a whole sequence h [T, width]; ``w`` maps the short names (in, conv, conv.b, dt_bias,
    A_log, D, norm, o) to tensors; ``m`` is the mixer's section of the document."""
    heads, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * P
    T = h.shape[0]
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, heads, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    y, _ = recurrence(x, B, C, softplus(dt + w["dt_bias"]), w["A_log"], w["D"])
    y = y.reshape(T, inner) * silu(z)
    y = group_norm(y, w["norm"], m["norm_groups"], eps)
    return y @ w["o"].T


def latent_of(h, w, eps):
    """The latent row per token that a latent-attention layer with a down-projection keeps."""
    return rms(h @ w["dkv"].T, eps) * w["dkv.norm"]


def latent_attention(h, c, w, m):
    """Softmax attention of the queries of h over keys and values that are up-projections of the latents c [T, kv_rank];
    a row sees itself and the ``mask.size`` - 1 rows before it (all earlier rows without a mask)."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    window = m["mask"]["size"] if m.get("mask") else None
    q = (h @ w["q"].T).reshape(T, H, D)
    k = (c @ w["uk"].T).reshape(T, H, D)
    v = (c @ w["uv"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=F)
    for i in range(T):
        first = 0 if window is None else max(0, i - window + 1)
        for head in range(H):
            scores = (k[first:i + 1, head] @ q[i, head]) * m["scale"]
            p = torch.softmax(scores, 0)
            out[i, head] = p @ v[first:i + 1, head]
    return out.reshape(T, H * V) @ w["o"].T


def expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, router, correction, top, scale):
    """(chosen experts [T, top], their weights [T, top])."""
    s = torch.sigmoid(h @ router.T)
    chosen = torch.topk(s + correction, top, dim=-1).indices
    kept = torch.gather(s, 1, chosen)
    return chosen, kept / (kept.sum(-1, keepdim=True) + 1e-20) * scale


def routed_experts(h, w, f):
    """``w``: short names (router, correction, e<j>.gate / up / down); ``f``: the feed-forward's section."""
    top, scale, limit = f["router"]["top"], f["router"].get("scale", 1.0), f["expert"]["limit"]
    chosen, weights = route(h, w["router"], w["correction"], top, scale)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(chosen[t, k])
            out[t] += weights[t, k] * expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)[0]
    return out


def token_side(x, tokens, table, layer, dim, w, eps, mult):
    """The per-layer token input: x + mult * rms(proj(gelu(gate x) * e)) * norm with e the layer's slice of the token's row."""
    e = table[tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w["gate"].T) * e) @ w["proj"].T
    return x + mult * rms(y, eps) * w["norm"]


def short_names(tensors, prefix):
    return {name[len(prefix):]: value.to(F) for name, value in tensors.items() if name.startswith(prefix)}


def forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence; with ``return_layers`` also the stream after every layer."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps, groups, mult = config["norm"]["eps"], config["norm"].get("groups", 1), config.get("residual_mult", 1.0)
    embed = tensors["embed"].to(F)
    x = embed[tokens]
    latents, after = {}, []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = group_norm(x, tensors[p + "norm1"].to(F), groups, eps)
        w = short_names(tensors, p + "mix.")
        if layer["type"] in ("mamba2", "mamba2_2"):
            y = mamba2(h, w, m, eps)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                latents[i] = latent_of(h, w, eps)
            y = latent_attention(h, latents[m["kv_from"] if m.get("kv_from") is not None else i], w, m)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            y = y + routed_experts(h, short_names(tensors, p + "mlp."), layer["mlp"])
        x = x + mult * y
        if config.get("token_side") is not None:
            x = token_side(x, tokens, tensors["side.embed"].to(F), i, config["token_side"]["dim"],
                           short_names(tensors, p + "side."), eps, mult)
        after.append(x)
    logits = group_norm(x, tensors["final.norm"].to(F), groups, eps) @ embed.T * config.get("logit_scale", 1.0)
    return (logits, torch.stack(after)) if return_layers else logits
