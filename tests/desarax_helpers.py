"""Small Desarax configurations and model folders for the tests.  None has the sizes of a real checkpoint; each makes
unequal what a convenient configuration would make equal or 1 (key and value widths of a head, the latent's width and the
heads' total, the windows of a layer and of the layer that reads its latents, groups of B and C and of the norms, the
filter's length, the chosen experts)."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

import plain_desarax as pd


def state_space(heads, vdim, state, groups, conv, norm_groups, second=False):
    return {"type": "mamba2_2" if second else "mamba2",
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def attention(heads, dim, vdim, kv_rank, window=None, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale if scale is not None else dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def moe(experts, top, ff, limit=1.0, scale=None):
    router = {"experts": experts, "top": top}
    if scale is not None:
        router["scale"] = scale
    return {"kind": "moe", "router": router, "expert": {"ff": ff, "limit": limit}}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(width, vocab, layers, groups=None, eps=1e-5, mult=None, logit_scale=None, side=None):
    doc = {"architecture": "Desarax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if groups is not None:
        doc["norm"]["groups"] = groups
    if mult is not None:
        doc["residual_mult"] = mult
    if logit_scale is not None:
        doc["logit_scale"] = logit_scale
    if side is not None:
        doc["token_side"] = {"dim": side}
    return doc


#: both kinds of state-space layer with different sizes; an attention layer whose latents a later layer reads with other
#: heads and a WIDER window than its own (the cache keeps what the wider one sees); an attention layer without a window and
#: without a feed-forward; the norm in three parts; windows of 24 and 37 positions over pages of 16 or 8
SMALL_A = config(48, 90, [
    layer(state_space(4, 12, 8, 2, 4, 2), moe(5, 2, 24, limit=0.7, scale=1.5)),
    layer(attention(3, 16, 8, 32, window=24, scale=0.3), moe(5, 2, 24, limit=0.7, scale=1.5)),
    layer(state_space(3, 8, 16, 1, 2, 3, second=True), moe(4, 1, 20, limit=2.0)),
    layer(attention(2, 8, 16, 32, window=37, kv_from=1), moe(5, 2, 24, limit=0.7, scale=1.5)),
    layer(attention(2, 24, 24, 16), None),
], groups=3, mult=0.6, logit_scale=1.5, side=10)
#: no table of the tokens' own inputs, the norm in one part, no factor on the residual or the logits, a filter of one
#: tap (the state keeps no inputs), every expert chosen, one head and one group, a window smaller than a page, a layer
#: that reads latents through no window although their own layer has one
SMALL_B = config(40, 70, [
    layer(attention(1, 24, 8, 24, window=5), moe(3, 3, 16)),
    layer(state_space(1, 24, 8, 1, 1, 1), None),
    layer(attention(4, 8, 8, 24, kv_from=0), moe(6, 2, 40, scale=0.5)),
    layer(state_space(6, 4, 4, 3, 5, 6, second=True), moe(3, 3, 16)),
], eps=1e-6)
#: no size is a multiple of eight (rows off 16-byte borders, ragged tiles in every kernel); a state that no lane count
#: divides; a window that is no multiple of a page
SMALL_C = config(36, 50, [
    layer(state_space(3, 10, 6, 3, 3, 5), moe(7, 3, 12, limit=0.5, scale=3.0)),
    layer(attention(3, 10, 6, 12, window=19), moe(3, 2, 20)),
    layer(attention(2, 6, 14, 12, window=7, kv_from=1), None),
    layer(state_space(2, 7, 20, 1, 4, 2, second=True), moe(5, 4, 12)),
], groups=2, mult=1.3, logit_scale=0.5, side=6)
#: sizes that the tensor-core kernels of the bfloat16 path take (latents of 64 and 32 entries), state-space heads of 64
#: columns over states of 128 and 64 entries, windows of 96 and of 50 positions, the per-token table wider than the stream
SMALL_D = config(64, 100, [
    layer(state_space(2, 64, 128, 1, 4, 2), moe(8, 2, 32)),
    layer(attention(4, 32, 32, 64, window=96), moe(8, 2, 32, limit=3.0, scale=2.5)),
    layer(attention(2, 64, 16, 64, window=50, kv_from=1), moe(8, 2, 32)),
    layer(state_space(4, 32, 64, 2, 3, 4, second=True), moe(8, 3, 48)),
    layer(attention(5, 16, 64, 32, window=130), moe(8, 2, 32)),
], groups=4, mult=0.8, logit_scale=2.5, side=72)


def spread(tensors: Dict[str, torch.Tensor], seed: int, sharpen: float = 8.0) -> Dict[str, torch.Tensor]:
    """Random-mode weights changed so that faults show: queries scaled up (peaked attention), decays from nearly none to
    fast with step sizes to match (a state that matters for hundreds of tokens beside one that forgets at once), filters,
    skips and projections of order one, routers that separate their experts, corrections that change the choice, expert
    matrices large enough that both clamps act, a per-token table of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for key, value in tensors.items():
        v, shape = value.float(), value.shape
        if key.endswith("mix.q"):
            v = v * sharpen
        elif key.endswith(("mix.in", "mix.dkv", "mix.uk", "mix.uv")):
            v = v * 8
        elif key.endswith("mix.A_log"):
            v = torch.rand(shape, generator=g) * 6 - 5          # decay rates exp(A_log) from 0.007 to 2.7
        elif key.endswith("mix.dt_bias"):
            v = torch.rand(shape, generator=g) * 4 - 3
        elif key.endswith(("mix.conv", "mix.conv.b")):
            v = torch.randn(shape, generator=g) * 0.5
        elif key.endswith("mix.D"):
            v = torch.randn(shape, generator=g)
        elif key.endswith("mlp.router"):
            v = v * 60
        elif key.endswith("mlp.correction"):
            v = torch.randn(shape, generator=g) * 0.3
        elif key.endswith((".gate", ".up")) and ".mlp.e" in key:
            v = v * 12
        elif key == "side.embed":
            v = v * 30
        elif key.endswith("side.gate"):
            v = v * 10
        out[key] = v
    return out


def make_folder(tmp_path, name: str, doc: dict, seed: int, dtype: torch.dtype, sharpen: float = 8.0) -> str:
    from sglang_rs_b200.weights import read_model_dir, write_file, write_model_folder
    folder = write_model_folder(str(tmp_path / name), doc, seed=seed, dtype=dtype)
    tensors = spread({k: v.clone() for k, v in read_model_dir(folder).items()}, seed, sharpen)
    write_file(os.path.join(folder, "model.safetensors"), {k: v.to(dtype) for k, v in tensors.items()})
    return folder


def load_folder(folder: str):
    from sglang_rs_b200.weights import read_model_dir
    with open(os.path.join(folder, "config.json")) as handle:
        doc = json.load(handle)
    return doc, read_model_dir(folder)


def random_requests(doc: dict, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(doc["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}


def oracle(folder: str, requests: Dict[str, List[int]]) -> Dict[str, np.ndarray]:
    doc, tensors = load_folder(folder)
    return {rid: pd.forward(doc, tensors, tokens).numpy() for rid, tokens in requests.items()}


def plain_greedy(doc, tensors, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(torch.argmax(pd.forward(doc, tensors, tokens)[-1])))
    return tokens[len(prompt):]


MARK = 41          # the token that the made-up models below look for
FILL = 40          # what stands where the mark would be, in sequences without it


def marked_folder(tmp_path, dtype: torch.dtype, mixer: str, window: Optional[int] = None, shared: bool = False,
                  wide: bool = False) -> str:
    """One or two layers that look for the one position holding ``MARK``.

    Only that token's embedding has an entry in channel 0; channel 1 is the same constant in every embedding.
    ``attention``: latent entry 0 reads channel 0; head 0's key and value read that entry, its query reads the constant,
    so the mark's score stands far above all others wherever it is visible.  With ``shared`` a second attention layer
    reads the first one's latents through a window twice as wide and looks for the mark in the same way.
    ``mamba``: head 0 decays by about 0.999 a token; its B and x read channel 0 (through the filter's current tap), its C
    reads the constant, so the state keeps the mark for hundreds of tokens and every later result holds it.  ``wide``:
    heads of 64 columns over states of 64 entries, the sizes at which prompt portions in bfloat16 run in parallel chunks."""
    from sglang_rs_b200.weights import read_model_dir, write_file
    if mixer == "attention":
        layers = [layer(attention(2, 16, 8, 16, window=window, scale=0.25), moe(3, 1, 8))]
        if shared:
            layers.append(layer(attention(3, 8, 8, 16, window=2 * window, kv_from=0, scale=0.35), None))
    else:
        P, N = (64, 64) if wide else (8, 8)
        layers = [layer(state_space(2, P, N, 1, 3, 1), moe(3, 1, 8))]
    doc = config(32, 60, layers, groups=1, mult=1.0, logit_scale=1.0)
    folder = make_folder(tmp_path, f"marked_{mixer}_{window}_{shared}_{wide}", doc, seed=7, dtype=dtype)
    t = {k: v.float().clone() for k, v in read_model_dir(folder).items()}
    t["embed"][:, 0] = 0
    t["embed"][MARK, 0] = 6.0
    t["embed"][:, 1] = 3.0
    for i in range(len(layers)):
        t[f"l{i}.norm1"][:] = 1.0
    if mixer == "attention":
        t["l0.mix.dkv"][0] = 0
        t["l0.mix.dkv"][0, 0] = 4.0
        t["l0.mix.dkv"][1:, 0] = 0
        t["l0.mix.dkv.norm"][:] = 1.0
        for i, dim in ((0, 16), (1, 8))[:len(layers)]:
            p = f"l{i}.mix."
            t[p + "uk"][:, 0] = 0
            t[p + "uk"][dim - 1] = 0
            t[p + "uk"][dim - 1, 0] = 4.0                        # head 0's last key entry reads latent entry 0
            t[p + "q"][dim - 1] = 0
            t[p + "q"][dim - 1, 1] = 6.0
            t[p + "uv"][:8] = 0
            t[p + "uv"][:8, 0] = 3.0
            t[p + "o"][:, :8] *= 10.0
    else:
        inner = 2 * P
        w = t["l0.mix.in"]
        w[inner:inner + P] = 0                                    # head 0's x
        w[inner:inner + P, 0] = 1.0
        w[2 * inner:2 * inner + N] = 0                            # B
        w[2 * inner:2 * inner + N, 0] = 1.0
        w[2 * inner + N:2 * inner + 2 * N] = 0                    # C
        w[2 * inner + N:2 * inner + 2 * N, 1] = 1.0
        w[2 * inner + 2 * N] = 0                                  # head 0's step size: softplus(0) everywhere
        conv, bias = t["l0.mix.conv"], t["l0.mix.conv.b"]
        for rows in (slice(0, P), slice(inner, inner + 2 * N)):
            conv[rows] = 0
            conv[rows, -1] = 1.0
            bias[rows] = 0
        t["l0.mix.A_log"][0], t["l0.mix.dt_bias"][0], t["l0.mix.D"][0] = -6.5, 0.0, 0.0
        t["l0.mix.A_log"][1], t["l0.mix.dt_bias"][1] = 0.5, 0.0
        t["l0.mix.norm"][:] = 1.0
        t["l0.mix.o"][:, :P] *= 10.0
    write_file(os.path.join(folder, "model.safetensors"), {k: v.to(dtype) for k, v in t.items()})
    return folder


def assert_rows_close(rows, expected, tolerance, dtype_name, what=""):
    """32-bit: every row within ``tolerance`` (largest difference over the largest |logit|).  bfloat16: a router's close
    call can go the other way once its input is rounded to 8 bits, which changes that row by far more than rounding does
    elsewhere; so there the rule is on the set of rows: at least 97 in 100 within ``tolerance`` and the median within a
    third of it.  A fault of a mechanism (a lost state, a key missed, a stale page) moves most rows and fails both."""
    errors, where = [], []
    for rid, by_pos in rows.items():
        scale = float(np.abs(expected[rid]).max())
        for pos, row in sorted(by_pos.items()):
            error = float(np.abs(row.astype(np.float64) - expected[rid][pos]).max()) / scale
            errors.append(error if np.isfinite(error) else float("inf"))
            where.append((rid, pos))
    errors = np.asarray(errors)
    worst = int(np.argmax(errors))
    if dtype_name == "float32":
        assert errors[worst] <= tolerance, (what, where[worst], float(errors[worst]))
        return
    over = int((errors > tolerance).sum())
    assert over <= 0.03 * len(errors) and float(np.median(errors)) <= tolerance / 3, \
        (what, over, len(errors), float(np.median(errors)), where[worst], float(errors[worst]))
